"""The kernels behind the parallel blocks, each by itself against a plain PyTorch float32 (or float64) statement of the same
operation: RMS norm in groups, token shift with state (alone and in one launch with the norm), xIELU, the gated side input, the
latent row store and the queries' rotation, the products per head on both kinds of units, and attention over latent rows in
32-bit and on the tensor cores (whole keys and keys cut into parts), with windows, pages in scrambled order and unequal requests."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_puzutar as plain

pytestmark = pytest.mark.gpu


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=dtype).cuda()


def layout(lengths):
    q_start = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    tok_seq = np.concatenate([np.full(n, i) for i, n in enumerate(lengths)]).astype(np.int32)
    return dev(tok_seq, torch.int32), dev(q_start, torch.int32)


@pytest.mark.parametrize("width, groups", [(96, 3), (200, 1), (64, 64), (1024, 2)])
def test_rms_norm_in_groups(width, groups):
    from liyab_b200 import ops
    rng = np.random.default_rng(width)
    x, w = rng.normal(0, 3, (9, width)), rng.normal(1, 0.3, width)
    rows = np.array([8, 0, 3, 3], dtype=np.int32)
    want = plain.grouped_rms_norm(x, w, groups, 1e-5)
    got = ops.rms_groups(dev(x), dev(w), groups, 1e-5, torch.empty(9, width, device="cuda"))
    assert np.abs(got.cpu().numpy() - want).max() < 2e-5
    got = ops.rms_groups(dev(x), dev(w), groups, 1e-5, torch.empty(4, width, dtype=torch.bfloat16, device="cuda"), dev(rows, torch.int32))
    assert np.abs(got.float().cpu().numpy() - want[rows]).max() < 3e-2


@pytest.mark.parametrize("fused", [False, True])
def test_token_shift_keeps_each_requests_last_row(fused):
    """Three requests in two steps (portions of 5, 1, 3 then 2, 1, 1) through slots 2, 0, 1: the second step's first rows blend
    with what the first step left; the plain statement runs over each request's whole sequence."""
    from liyab_b200 import ops
    rng = np.random.default_rng(3)
    width, groups = 48, 4
    w, mu = rng.normal(1, 0.2, width), rng.uniform(0, 1, width)
    seqs = [rng.normal(0, 2, (n, width)) for n in (7, 2, 4)]
    want = [plain.token_shift(plain.grouped_rms_norm(s, w, groups, 1e-5), mu) for s in seqs]
    state = torch.zeros(3, width, device="cuda")
    slots = dev([2, 0, 1], torch.int32)
    at = [0, 0, 0]
    for lengths in ([5, 1, 3], [2, 1, 1]):
        x = np.concatenate([s[a:a + n] for s, a, n in zip(seqs, at, lengths)])
        tok_seq, q_start = layout(lengths)
        h, out = torch.empty(len(x), width, device="cuda"), torch.empty(len(x), width, device="cuda")
        if fused:
            ops.token_shift(h, dev(mu), out, state, tok_seq, q_start, slots, x=dev(x), weight=dev(w), groups=groups, eps=1e-5)
        else:
            ops.rms_groups(dev(x), dev(w), groups, 1e-5, h)
            ops.token_shift(h, dev(mu), out, state, tok_seq, q_start, slots)
        ref = np.concatenate([r[a:a + n] for r, a, n in zip(want, at, lengths)])
        assert np.abs(out.cpu().numpy() - ref).max() < 2e-5
        at = [a + n for a, n in zip(at, lengths)]


def test_xielu():
    from liyab_b200 import ops
    z = np.linspace(-12, 12, 7 * 331).reshape(7, 331)
    for p, q in ((0.3, -0.7), (-2.0, 1.5)):
        want = plain.xielu(z, p, q)
        got = ops.xielu(dev(z), dev([p, q]))
        assert np.abs(got.cpu().numpy() - want).max() < 1e-4 * np.abs(want).max()
        z16 = dev(z[:, :328], torch.bfloat16)
        want16 = plain.xielu(z16.float().cpu().numpy().astype(np.float64), p, q)
        assert np.abs(ops.xielu(z16, dev([p, q])).float().cpu().numpy() - want16).max() < 8e-3 * np.abs(want16).max()


@pytest.mark.parametrize("width, dim", [(96, 8), (100, 3), (256, 64)])
def test_gated_side_input(width, dim):
    from liyab_b200 import ops
    rng = np.random.default_rng(dim)
    x, tokens = rng.normal(0, 2, (11, width)), rng.integers(0, 30, 11)
    W = {"side.embed": rng.normal(0, 1, (30, 2 * dim)), "l1.side.gate": rng.normal(0, width ** -0.5, (dim, width)),
         "l1.side.proj": rng.normal(0, 1, (width, dim)), "l1.side.norm": rng.normal(0.5, 0.2, width)}
    want = plain.token_side(x, tokens, W, 1, dim, 1e-5)
    got = ops.token_side(dev(x), dev(tokens, torch.int32), dev(W["side.embed"][:, dim:].copy()), dev(W["l1.side.gate"]), dev(W["l1.side.proj"]),
                         dev(W["l1.side.norm"]), 1e-5)
    assert np.abs(got.cpu().numpy() - want).max() < 3e-5 * np.abs(want).max()


def latent_case(seed, H, dim, rot, rot_dims, rank, window, lengths, pasts, page, base=1e4):
    """Random queries, latent rows at scrambled pages, and the float64 result: (inputs ..., attended latents [T, H, rank])."""
    rng = np.random.default_rng(seed)
    D = rank + rot
    S = len(lengths)
    total = [p + n for p, n in zip(pasts, lengths)]
    n_pages = sum(-(-t // page) for t in total) + 3
    order = rng.permutation(n_pages)
    width = max(-(-t // page) for t in total)
    table = np.full((S, width), -1, dtype=np.int32)
    rows = np.zeros((n_pages * page, D))
    seqs = []
    at = 0
    for s in range(S):
        c = rng.normal(0, 1, (total[s], D))
        seqs.append(c)
        for j in range(-(-total[s] // page)):
            table[s, j] = order[at]
            at += 1
        for pos in range(total[s]):
            rows[table[s, pos // page] * page + pos % page] = c[pos]
    T = sum(lengths)
    wide = rng.normal(0, 1, (T, H, D))
    positions = np.concatenate([np.arange(p, p + n) for p, n in zip(pasts, lengths)]).astype(np.int32)
    scale = 0.6 / math.sqrt(D)
    want = np.zeros((T, H, rank))
    t = 0
    for s in range(S):
        for i in range(lengths[s]):
            p = positions[t]
            lo = max(0, p - window + 1) if window else 0
            keys = seqs[s][lo:p + 1]
            sc = np.einsum("hd,jd->hj", wide[t], keys) * scale
            sc -= sc.max(axis=1, keepdims=True)
            w = np.exp(sc)
            w /= w.sum(axis=1, keepdims=True)
            want[t] = w @ keys[:, :rank]
            t += 1
    return wide, rows, table, positions, scale, want


@pytest.mark.parametrize("H, rank, rot, window, page", [(3, 40, 8, 20, 16), (5, 160, 32, 0, 16), (6, 128, 16, 50, 64), (1, 24, 0, 1, 16)])
def test_latent_attention_32_bit(H, rank, rot, window, page):
    from liyab_b200 import ops
    lengths, pasts = [37, 1, 5, 1], [0, 130, 60, 15]
    wide, rows, table, positions, scale, want = latent_case(rank, H, 0, rot, rot, rank, window, lengths, pasts, page)
    tok_seq, q_start = layout(lengths)
    out = torch.empty(sum(lengths), H * rank, device="cuda")
    ops.latent_attention(dev(wide.reshape(len(wide), -1)), dev(rows), tok_seq, dev(positions, torch.int32), q_start, dev(pasts, torch.int32),
                         dev(table, torch.int32), out, H, rank, rot, page, scale, window)
    assert np.abs(out.cpu().numpy().reshape(want.shape) - want).max() < 2e-5


@pytest.mark.parametrize("H, rank, rot, window, page, lengths, pasts, splits", [
    (12, 64, 16, 40, 16, [70, 1, 9], [0, 200, 33], 1),
    (20, 96, 32, 0, 16, [33, 2], [5, 90], 1),
    (2, 256, 16, 100, 64, [130], [0], 1),
    (4, 512, 64, 45, 16, [50, 3], [0, 61], 1),
    (12, 256, 16, 512, 16, [1, 1, 1, 1, 1], [700, 3, 511, 512, 64], 5),
    (3, 32, 16, 33, 16, [1, 1], [32, 100], 2),
])
def test_latent_attention_on_tensor_cores(H, rank, rot, window, page, lengths, pasts, splits):
    """bfloat16 operands: the float64 result is made from the rounded queries and rows, so what is left is the rounding of the
    weights and the accumulation."""
    from liyab_b200 import ops
    wide, rows, table, positions, scale, _ = latent_case(7 * rank + H, H, 0, rot, rot, rank, window, lengths, pasts, page)
    wide16, rows16 = dev(wide.reshape(len(wide), -1), torch.bfloat16), dev(rows, torch.bfloat16)
    # the same case with the rounded values as the truth
    D = rank + rot
    T = sum(lengths)
    w64, r64 = wide16.float().cpu().numpy().astype(np.float64).reshape(T, H, D), rows16.float().cpu().numpy().astype(np.float64)
    want = np.zeros((T, H, rank))
    t = 0
    for s, (n, past) in enumerate(zip(lengths, pasts)):
        for i in range(n):
            p = past + i
            lo = max(0, p - window + 1) if window else 0
            keys = np.stack([r64[table[s, j // page] * page + j % page] for j in range(lo, p + 1)])
            sc = np.einsum("hd,jd->hj", w64[t], keys) * scale
            sc -= sc.max(axis=1, keepdims=True)
            w = np.exp(sc)
            w /= w.sum(axis=1, keepdims=True)
            want[t] = w @ keys[:, :rank]
            t += 1
    tok_seq, q_start = layout(lengths)
    out = torch.full((T, H * rank), float("nan"), device="cuda")
    ops.latent_attention(wide16, rows16, tok_seq, dev(positions, torch.int32), q_start, dev(pasts, torch.int32), dev(table, torch.int32), out, H, rank,
                         rot, page, scale, window, tensor_cores=True, n_splits=splits)
    err = np.abs(out.cpu().numpy().reshape(want.shape) - want).max()
    assert err < 2e-2, err


@pytest.mark.parametrize("M", [5, 70])
def test_products_per_head(M):
    """Keys' maps onto queries (rows of the map along n) and values' maps onto attended latents (rows along k), on the 32-bit units
    and on the tensor cores."""
    from liyab_b200 import ops
    rng = np.random.default_rng(M)
    H, dim, rot, rank, vdim = 3, 24, 8, 64, 40
    q = rng.normal(0, 1, (M, H, dim + rot))
    uk = rng.normal(0, 1, (H, dim, rank))
    uv = rng.normal(0, 1, (H, vdim, rank))
    att = rng.normal(0, 1, (M, H, rank))
    for tensor in (False, True):
        bdt = torch.bfloat16 if tensor else torch.float32
        tol = 3e-2 if tensor else 1e-4
        uk_d, uv_d = dev(uk, bdt), dev(uv, bdt)
        wide = torch.zeros(M, H * (rank + rot), dtype=bdt, device="cuda")
        ops.head_matmul(dev(q.reshape(M, -1)), dim + rot, uk_d.reshape(-1), dim * rank, rank, 1, wide, rank + rot, rank, dim, H, tensor_cores=tensor)
        want = np.einsum("mhd,hdn->mhn", q[..., :dim], uk_d.float().cpu().numpy().astype(np.float64))
        got = wide.float().cpu().numpy().reshape(M, H, rank + rot)
        assert np.abs(got[..., :rank] - want).max() < tol * np.abs(want).max() and np.abs(got[..., rank:]).max() == 0
        values = torch.zeros(M, H * vdim, dtype=bdt, device="cuda")
        ops.head_matmul(dev(att.reshape(M, -1)), rank, uv_d.reshape(-1), vdim * rank, 1, rank, values, vdim, vdim, rank, H, tensor_cores=tensor)
        want = np.einsum("mhr,hvr->mhv", att, uv_d.float().cpu().numpy().astype(np.float64))
        assert np.abs(values.float().cpu().numpy().reshape(M, H, vdim) - want).max() < tol * np.abs(want).max()


def test_latent_store_and_rotation():
    from liyab_b200 import ops
    rng = np.random.default_rng(2)
    T, H, dim, rank, rot, rot_dims, base = 6, 3, 8, 24, 12, 8, 300.0
    d = rng.normal(0, 2, (T, rank + rot))
    gain = rng.normal(1, 0.2, rank)
    positions = np.array([0, 1, 77, 1000, 5, 64], dtype=np.int32)
    slots = np.array([9, 3, -1, 0, 4, 5], dtype=np.int32)
    freq = np.array([base ** (-2.0 * i / rot_dims) for i in range(rot_dims // 2)])
    cache = torch.zeros(10, rank + rot, device="cuda")
    ops.latent_store(dev(d), dev(gain), dev(freq), dev(positions, torch.int32), dev(slots, torch.int32), cache, rank, rot, rot_dims, 1e-5)
    got = cache.cpu().numpy()
    c = plain.rms(d[:, :rank], 1e-5) * gain
    kr = plain.rotate_half(d[:, rank:], positions, base, rot_dims)
    for t in range(T):
        if slots[t] >= 0:
            assert np.abs(got[slots[t], :rank] - c[t]).max() < 1e-5 and np.abs(got[slots[t], rank:] - kr[t]).max() < 2e-4
    assert np.abs(got[[1, 2, 6, 7, 8]]).max() == 0          # a negative slot writes nowhere
    q = rng.normal(0, 1, (T, H, dim + rot))
    wide = torch.zeros(T, H * (rank + rot), device="cuda")
    ops.rope_heads(dev(q.reshape(T, -1)), dev(freq), dev(positions, torch.int32), wide, H, dim, rot, rot_dims, rank)
    want = plain.rotate_half(q[..., dim:], positions, base, rot_dims)
    got = wide.cpu().numpy().reshape(T, H, rank + rot)
    assert np.abs(got[..., rank:] - want).max() < 2e-4 and np.abs(got[..., :rank]).max() == 0


@pytest.mark.parametrize("m, n, k", [(5, 136, 96), (40, 200, 128), (300, 256, 192), (9, 264, 2048)])
def test_xielu_in_the_products_epilogues(m, n, k):
    """The activation inside every product kernel that can take the shape (its two learned numbers behind the bias) against the
    product in float64 followed by the plain activation."""
    from liyab_b200 import ops
    rng = np.random.default_rng(m)
    a, w = rng.normal(0, 1, (m, k)), rng.normal(0, k ** -0.5, (n, k))
    bias, pq = rng.normal(0, 0.3, n), np.array([0.4, -0.8])
    joined = dev(np.concatenate([bias, pq]))
    a16, w16 = dev(a, torch.bfloat16), dev(w, torch.bfloat16)
    want32 = plain.xielu(a @ w.T + bias, *pq)
    want16 = plain.xielu(a16.double().cpu().numpy() @ w16.double().cpu().numpy().T + bias, *pq)
    scale = np.abs(want32).max()
    out = ops.gemm_ffma(dev(a), dev(w), joined, torch.empty(m, n, device="cuda"), m, "xielu")
    assert np.abs(out.cpu().numpy() - want32).max() < 2e-5 * scale
    ran = 0
    for out_dtype, tol in ((torch.float32, 2e-4), (torch.bfloat16, 1e-2)):
        if ops.gemm_rows_supports(a16, w16, m):
            out = ops.gemm_rows(a16, w16, joined, torch.empty(m, n, dtype=out_dtype, device="cuda"), m, "xielu")
            assert np.abs(out.float().cpu().numpy() - want16).max() < tol * scale
            ran += 1
        if ops.tcgen05_accepts(a16, w16):
            out = torch.empty(m, n, dtype=out_dtype, device="cuda")
            if m > 64 and ops.gemm_persistent_tile(a16, w16, out, m) > 0:
                ops.gemm_persistent(a16, w16, joined, out, m, "xielu")
            else:
                ops.linear(a16, w16, joined, out, m, "xielu")
            assert np.abs(out.float().cpu().numpy() - want16).max() < tol * scale
            ran += 1
            splits = ops.gemm_splits(m, n, k)
            if m <= 64 and splits > 1:       # K split over blocks: the activation sits in the second launch, which adds the parts
                partial = torch.empty(splits * m * n, device="cuda")
                counters = torch.zeros(-(-n // 128), dtype=torch.int32, device="cuda")
                out = ops.gemm_tcgen05(a16, w16, joined, torch.empty(m, n, dtype=out_dtype, device="cuda"), m, "xielu", None, 0, partial, counters, splits)
                assert np.abs(out.float().cpu().numpy() - want16).max() < tol * scale
                ran += 1
    assert ran >= 2
