"""Vosurax in the engine against the plain implementation (plain_vosurax.py): every mechanism by itself through the
parts' taps, then whole prompts, token-by-token decoding, portions down to two tokens, mixed batches with pages and
state slots used again, keys at the chunks' edges and at page borders, memories that reach far back, the first tokens
of a sequence, long decoding, and greedy generation through the engine's own entry point and scheduler."""
from __future__ import annotations

import copy
import os
import subprocess

import numpy as np
import pytest

import plain_vosurax as plain
import trace_tools as tt
from vosurax_models import CONFIGS, dense, layer, model_folder, moe, random_weights, retention, side_by_side, write_model

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# float32: largest |engine - plain| on a logit as a fraction of the largest |logit| of the sequence.
REL_TOL = 1e-4
LENGTHS = {"A": [150, 70, 33, 21, 7, 2, 1, 45], "B": [140, 72, 64, 1, 2, 97, 40], "C": [120, 47, 2, 64, 1, 33], "D": [100, 33, 32, 31, 2, 65]}


def tokens_of(name, i, n):
    config, seed = CONFIGS[name]
    return np.random.default_rng(1000 * seed + i).integers(0, config["vocab"], size=n).astype(int).tolist()


def request_set(name):
    return {f"r{i}": tokens_of(name, i, n) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = str(tmp_path_factory.mktemp("vosurax"))
    return {name: model_folder(base, name) for name in CONFIGS}


@pytest.fixture(scope="module")
def oracle(models):
    return {name: {r: plain.forward(config, weights, toks) for r, toks in request_set(name).items()}
            for name, (_, config, weights) in models.items()}


def make_engine(path, dtype, max_tokens, **options):
    from liyab_b200.engine import Replayer
    options.setdefault("max_requests", 4)
    return Replayer(path, dtype, max_tokens, **options)


def check(got, want, dtype, rel_tol=REL_TOL, flips=True):
    """float32: every logit within rel_tol of the plain model's.  bfloat16: per row, the root mean square of the
    difference (its mean taken off) over that of the sequence's logits; 8 bits of mantissa put it near a percent, and the
    median is held to 1.5 %, the mean to 2 %.  Where two experts' scores lie close, a rounding sends a row to another expert, and the memories
    carry that difference to the positions after it (`flips`): then up to a tenth of the rows may lie beyond 6 %, none beyond
    the logits' own spread, and the mean is held to 4 %.  Models whose routers decide by clear margins are held to 6 % in every row."""
    if dtype != "bfloat16":
        return tt.check_rows(got, want, rel_tol)
    errs = []
    for (r, pos), row in got.items():
        d = row.astype(np.float64) - want[r][pos]
        spread = want[r] - want[r].mean(axis=-1, keepdims=True)
        errs.append(np.sqrt(((d - d.mean()) ** 2).mean()) / np.sqrt((spread ** 2).mean()))
    errs = np.asarray(errs)
    assert np.isfinite(errs).all() and np.median(errs) <= 1.5e-2, f"median relative error {np.median(errs):.3e}"
    if flips:
        assert errs.mean() <= 4e-2, f"mean relative error {errs.mean():.3e}"
        assert (errs > 6e-2).mean() <= 0.10 and errs.max() < 1.0, f"{(errs > 6e-2).sum()} of {len(errs)} rows are off by more than 6 %, the worst by {errs.max():.2f}"
    else:
        assert errs.mean() <= 2e-2 and errs.max() <= 6e-2, f"mean {errs.mean():.3e}, {(errs > 6e-2).sum()} of {len(errs)} rows are off by more than 6 %"
    return {"mean": float(errs.mean()), "worst": float(errs.max())}


# What the plain model calls a part's output -> the name of the engine's tap.
TAPS = {"retention.heads": "memory", "memory.heads": "memory", "left": "branch.left", "right": "branch.right", "mixer": "mixer", "routed": "routed",
        "out": "block"}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_every_mechanism_by_itself(name, models):
    """The parts' outputs, run by run, against the plain functions in float32: the memories' heads before their norm,
    each branch of a side-by-side mixer, the stream after the mixer, after the routed experts and after the block
    (so the pass offsets, the norms with gains around zero and both feed-forwards are in it).  A whole prompt, then the
    same prompt cut in two and in three (state and cache)."""
    from liyab_b200.engine import StepEntry
    path, config, weights = models[name]
    toks = tokens_of(name, 50, 45)
    want = []
    plain.forward(config, weights, toks, traces=want)
    for cuts in ([len(toks)], [19, len(toks)], [2, 33, len(toks)]):
        engine = make_engine(path, "float32", 128)
        runs = [dict() for _ in want]
        at = [-1]
        def tap(n, rows):
            if n == "pass_offset":
                return
            if n == "mixer_norm":       # a block's first tap
                at[0] += 1
            run = runs[at[0] % len(want)]
            run.setdefault(n, []).append(rows)
        engine.set_tap(tap)
        engine.cache.open("a")
        lo = 0
        for hi in cuts:
            engine.step([StepEntry("a", toks[lo:hi], [])])
            lo = hi
        assert at[0] + 1 == len(cuts) * len(want)
        for i, ref_run in enumerate(want):
            runs[i]["block"] = runs[i]["feed_forward" if "feed_forward" in runs[i] else "mixer"]      # the stream as the block leaves it
            for plain_name, tap_name in TAPS.items():
                if plain_name not in ref_run:
                    continue
                ref = ref_run[plain_name]
                rows = np.concatenate(runs[i][tap_name], axis=0)
                assert rows.shape == ref.shape, (plain_name, rows.shape, ref.shape)
                err = np.abs(rows - ref).max() / max(np.abs(ref).max(), 1e-30)
                assert err < 5e-5, f"{plain_name} of run {i} (cuts {cuts}): {err:.2e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_every_cutting_matches_plain(name, dtype, models, oracle):
    path, config, _ = models[name]
    reqs = request_set(name)
    want = oracle[name]
    n_rows = sum(len(t) for t in reqs.values())
    traces = {"whole": tt.whole(reqs), "one_by_one": tt.tail_one_by_one(reqs, 10 ** 6), "tail": tt.tail_one_by_one(reqs, 40),
              "portions": tt.changing_portions(reqs), "odd_portions": tt.changing_portions(reqs, sizes=(2, 31, 2, 17, 1, 3, 33, 16, 2))}
    for kind, steps in traces.items():
        engine = make_engine(path, dtype, max_tokens=256)
        got = tt.collect(engine, steps)
        assert len(got) == n_rows
        check(got, want, dtype)
    # Mixed batches over a pool for the trace's own peak and four state slots for all requests: pages and slots are used again.
    for seed in (3, 4):
        steps = tt.mixed(reqs, max_live=4, seed=seed)
        assert max(len(e) for e, _ in steps) >= 3
        engine = make_engine(path, dtype, max_tokens=tt.peak_tokens(steps, 64))
        got = tt.collect(engine, steps)
        assert len(got) == n_rows
        check(got, want, dtype)
        assert len(reqs) > 4 and engine.cache.state_slots_free() == 4


def test_batches_of_unequal_requests_match_each_alone(models):
    """The engine against itself: every request alone and all in mixed batches give the same logits up to rounding."""
    path, _, _ = models["A"]
    reqs = request_set("A")
    alone = tt.collect(make_engine(path, "float32", max_tokens=256), tt.whole(reqs))
    steps = tt.mixed(reqs, max_live=4, seed=11, portion=23)
    together = tt.collect(make_engine(path, "float32", max_tokens=tt.peak_tokens(steps, 64)), steps)
    assert alone.keys() == together.keys()
    scale = max(np.abs(r).max() for r in alone.values())
    assert max(np.abs(alone[k] - together[k]).max() for k in alone) / scale < 2e-5


@pytest.mark.parametrize("page_size", [16, 64])
def test_pages_of_other_sizes(page_size, models, oracle):
    path, _, _ = models["A"]
    engine = make_engine(path, "float32", max_tokens=512, page_size=page_size)
    got = tt.collect(engine, tt.changing_portions(request_set("A"), sizes=(63, 2, 1, 64, 17)))
    check(got, oracle["A"], "float32")


def sharp_model(base, chunk, kv_heads=1):
    """One side-by-side block whose attention branch has its scores sharpened so that one key takes nearly all the weight, and
    whose memory branch is turned down: a key that is wrongly seen or wrongly hidden moves the logits by far more than rounding."""
    config = dict(architecture="Vosurax", vocab=40, width=32, norm=dict(eps=1e-5), layers=[
        layer(side_by_side(2, kv_heads, 8, 12, 40.0, chunk, 1, 4, 4, 8.0), dense(40))])
    weights = random_weights(config, 77)
    weights["l0.mix.right.out"] = weights["l0.mix.right.out"] * 0.0625
    return write_model(os.path.join(base, f"sharp_{chunk}_{kv_heads}"), config, weights), config, weights


@pytest.mark.parametrize("chunk", [16, 17, 15, 33, 5, 64])
def test_chunk_edges_in_prompts_and_in_decoding(chunk, tmp_path):
    """Chunks that end on, just before and just after page borders; every position of a prompt and of decoding across many
    chunks' edges against the plain model; the plain model with a chunk one larger or one smaller, or with chunks counted from
    where a portion starts, must differ clearly (or the test shows nothing)."""
    path, config, weights = sharp_model(str(tmp_path), chunk, kv_heads=2 if chunk == 33 else 1)
    toks = np.random.default_rng(5).integers(0, config["vocab"], size=150).astype(int).tolist()
    want = plain.forward(config, weights, toks)
    for delta in (-1, 1):
        other = copy.deepcopy(config)
        other["layers"][0]["mixer"]["left"]["mask"]["size"] += delta
        moved = np.abs(plain.forward(other, weights, toks) - want).max(axis=1) / np.abs(want).max()
        assert (moved > 1e-2).sum() >= 5, "the weights do not show a chunk that is one off"
    reqs = {"a": toks}
    for steps in (tt.whole(reqs), tt.tail_one_by_one(reqs, 110), tt.changing_portions(reqs, sizes=(15, 2, 16, 17, 1, 33, 7))):
        for dtype, tol in (("float32", 1e-4), ("bfloat16", None)):
            engine = make_engine(path, dtype, max_tokens=192)
            got = tt.collect(engine, steps)
            if tol is not None:
                tt.check_rows(got, {"a": want}, tol)
            else:
                errs = np.array([np.abs(row - want[pos]).max() for (_, pos), row in got.items()]) / np.abs(want).max()
                assert np.median(errs) < 2e-2 and (errs > 0.15).mean() < 0.05, (np.median(errs), errs.max())
    # The attention's cache unit keeps what a chunk can see, no more: pages behind the chunk came back.
    from liyab_b200.engine import StepEntry
    engine = make_engine(path, "float32", max_tokens=192)
    engine.cache.open("a")
    engine.step([StepEntry("a", toks, [])])
    assert sum(engine.cache.pages_in_use().values()) <= (chunk + 15) // 16 + 1


def long_memory_model(base, kind):
    """One block whose memory forgets slowly (a decay just under one; a forget gate pushed open), so that tokens hundreds of
    positions back still carry weight."""
    if kind == "retention":
        config = dict(architecture="Vosurax", vocab=50, width=32, norm=dict(eps=1e-5), layers=[layer(retention(2, 8, 12, [0.9995, 0.998], 8, 1e4), dense(40))])
        weights = random_weights(config, 5)
    else:
        config = dict(architecture="Vosurax", vocab=50, width=32, norm=dict(eps=1e-5), layers=[layer(side_by_side(1, 1, 4, 4, 0.5, 8, 2, 8, 12, 14.0), dense(40))])
        weights = random_weights(config, 6)
        weights["l0.mix.right.f.b"] = weights["l0.mix.right.f.b"] * 0.0 + 9.0
        weights["l0.mix.left.out"] = weights["l0.mix.left.out"] * 0.0625
    return write_model(os.path.join(base, f"long_{kind}"), config, weights), config, weights


@pytest.mark.parametrize("kind", ["retention", "gated"])
def test_memories_reach_far_back(kind, tmp_path):
    """420 tokens through a memory that forgets slowly: whole, decoded, in portions that end on and off page borders.  A memory
    that lost its first 200 tokens gives clearly different logits (shown on the plain model)."""
    path, config, weights = long_memory_model(str(tmp_path), kind)
    toks = np.random.default_rng(9).integers(1, 50, size=420).astype(int).tolist()
    want = plain.forward(config, weights, toks)
    lost = plain.forward(config, weights, toks[200:])
    assert (np.abs(lost - want[200:]).max(axis=1) / np.abs(want).max() > 1e-2).sum() >= 100, "the weights do not show a lost state"
    reqs = {"a": toks}
    for steps in (tt.whole(reqs), tt.tail_one_by_one(reqs, 30), tt.changing_portions(reqs, sizes=(255, 2, 64, 1, 17))):
        got = tt.collect(make_engine(path, "float32", max_tokens=448), steps)
        tt.check_rows(got, {"a": want}, 2e-4)


def test_first_tokens_of_a_sequence(tmp_path):
    """Input gates far below zero at a sequence's start: the running maximum stays near its starting value 0, little has been taken
    into the memory, and what divides the read-out is the floor exp(-m), not |n . q|.  Without the floor the plain model answers
    clearly differently, so a floor that is left out, or a maximum or a state that does not start at zero, shows."""
    config = dict(architecture="Vosurax", vocab=50, width=32, norm=dict(eps=1e-5), layers=[layer(side_by_side(1, 1, 4, 4, 0.5, 8, 2, 8, 12, 14.0), dense(40))])
    weights = random_weights(config, 8)
    weights["l0.mix.right.i.b"] = weights["l0.mix.right.i.b"] * 0.0 - 6.0
    weights["l0.mix.left.out"] = weights["l0.mix.left.out"] * 0.0625
    path = write_model(str(tmp_path / "first"), config, weights)
    toks = np.random.default_rng(3).integers(0, 50, size=40).astype(int).tolist()
    want = plain.forward(config, weights, toks)
    plain.FLOOR = False
    try:
        other = plain.forward(config, weights, toks)
    finally:
        plain.FLOOR = True
    assert (np.abs(other - want).max(axis=1) / np.abs(want).max() > 1e-2).sum() >= 5, "the weights do not show the divisor's floor"
    reqs = {"a": toks}
    for steps in (tt.whole(reqs), tt.tail_one_by_one(reqs, 10 ** 6), tt.changing_portions(reqs, sizes=(2, 3, 2, 17))):
        got = tt.collect(make_engine(path, "float32", max_tokens=64), steps)
        tt.check_rows(got, {"a": want}, 1e-4)


def test_sharp_router_and_weight_on_the_input(tmp_path):
    """Experts chosen by clear margins (a large router), one and several a row: the engine picks the plain model's experts in both
    types, and the weight acts on the expert's input (scaling its output instead changes the plain model's logits clearly)."""
    config = dict(architecture="Vosurax", vocab=60, width=48, norm=dict(eps=1e-5), layers=[
        layer(retention(2, 8, 8, [0.9, 0.8], 4), moe(7, 3, 24, 0)), layer(retention(1, 8, 8, [0.9], 0), moe(5, 1, 16, 8))])
    weights = random_weights(config, 12, router_std=12.0)
    path = write_model(str(tmp_path / "router"), config, weights)
    toks = np.random.default_rng(27).integers(0, 60, size=48).astype(int).tolist()
    traces = []
    want = plain.forward(config, weights, toks, traces=traces)
    for trace, l in zip(traces, config["layers"]):       # the last chosen expert and the best unchosen one are clearly apart
        sc, top = trace["scores"], l["mlp"]["router"]["top"]
        z = -np.sort(-(np.log(sc) - np.log1p(-sc)), axis=1)
        assert np.nanmin(z[:, top - 1] - z[:, top]) > 0.3, "the router's margins are not clear"
    real = plain.routed_ff

    def weight_on_output(h, W, p, mlp, trace=None):
        s = plain.sigmoid(h @ W[p + "router"].T)
        order = np.argsort(-s, axis=1, kind="stable")[:, :mlp["router"]["top"]]
        y = np.zeros((h.shape[0], W[p + "e0.down"].shape[0]))
        for t in range(h.shape[0]):
            for e in order[t]:
                y[t] += s[t, e] * plain.gated_ff(h[t:t + 1], W, f"{p}e{e}.")[0]
        return y + (plain.gated_ff(h, W, p + "shared.") if mlp.get("shared") else 0.0)

    plain.routed_ff = weight_on_output
    try:
        other = plain.forward(config, weights, toks)
    finally:
        plain.routed_ff = real
    assert np.abs(other - want).max() / np.abs(want).max() > 1e-2
    for dtype in ("float32", "bfloat16"):
        for steps in (tt.whole({"a": toks}), tt.changing_portions({"a": toks}, sizes=(20, 1, 2, 9))):
            check(tt.collect(make_engine(path, dtype, max_tokens=128), steps), {"a": want}, dtype, flips=False)


def test_long_decoding_reuses_pages(models):
    """Decoding one token at a time far past every chunk: pages are freed behind the chunks and handed out again, and the
    memories run through 400 single steps."""
    path, config, weights = models["A"]
    toks = tokens_of("A", 99, 400)
    want = plain.forward(config, weights, toks)
    engine = make_engine(path, "float32", max_tokens=128)       # far fewer pages than 400 positions
    got = tt.collect(engine, tt.tail_one_by_one({"a": toks}, 395))
    assert len(got) == 400
    tt.check_rows(got, {"a": want}, 2e-4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, models, oracle, tmp_path):
    path, config, _ = models["A"]
    reqs = request_set("A")
    steps = tt.mixed(reqs, max_live=4, seed=8)
    out_dir = str(tmp_path / "out")
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", path, "--dtype", dtype, "--out", out_dir,
                           "--max-tokens", str(tt.peak_tokens(steps))], input=tt.to_jsonl(steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    held, got = {}, {}
    for i, (entries, end) in enumerate(steps):
        data = np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(-1, config["vocab"])
        row = 0
        for r, toks, want in entries:
            base = held.get(r, 0)
            for w in want:
                got[(r, base + w)] = data[row]
                row += 1
            held[r] = base + len(toks)
        assert row == data.shape[0]
    check(got, oracle["A"], dtype)


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(graphs, models):
    """Prompts of unequal length served together by the scheduler, greedy, against the plain model's own greedy
    continuation (compared while the plain model's best two logits are clearly apart)."""
    from liyab_b200.engine import Engine
    from liyab_b200.sampling import SamplingParams
    path, config, weights = models["A"]
    prompts = [tokens_of("A", 70 + i, n) for i, n in enumerate((37, 5, 1, 64, 18, 90))]
    engine = Engine(model=path, dtype="float32", context_length=256, max_requests=4, max_batched_tokens=48, cuda_graphs=graphs)
    results = engine.generate_batch(prompts, SamplingParams(max_tokens=24, temperature=0.0))
    engine.close()
    for prompt, res in zip(prompts, results):
        assert res.error is None and len(res.tokens) == 24
        seq = list(prompt)
        for tok in res.tokens:
            row = plain.forward(config, weights, seq)[-1]
            best = np.sort(row)[-2:]
            if best[1] - best[0] < 1e-3 * np.abs(row).max():
                break
            assert tok == int(np.argmax(row))
            seq.append(tok)


def test_command_line_and_sampling(models):
    """The command line generates greedily what the plain model would, and the engine's sampler with a seed gives the same
    tokens twice and other tokens with another seed."""
    import json
    from liyab_b200.engine import Engine
    from liyab_b200.sampling import SamplingParams
    path, config, weights = models["B"]
    prompt = tokens_of("B", 90, 9)
    cmd = [os.path.join(ROOT, "bin", "liyab-cli"), "-m", path, "-p", ",".join(map(str, prompt)), "-n", "8", "--temp", "0", "--dtype", "float32",
           "--ctx", "128", "--json"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")]
    seq = list(prompt)
    for tok in lines[1]["tokens"]:
        row = plain.forward(config, weights, seq)[-1]
        best = np.sort(row)[-2:]
        if best[1] - best[0] < 1e-3 * np.abs(row).max():
            break
        assert tok == int(np.argmax(row))
        seq.append(tok)
    draws = []
    for seed in (5, 5, 6):
        engine = Engine(model=path, dtype="bfloat16", context_length=128, max_requests=4)
        draws.append(engine.generate_tokens(prompt, SamplingParams(max_tokens=12, temperature=0.9, top_k=20, top_p=0.95, seed=seed)).tokens)
        engine.close()
    assert draws[0] == draws[1] and draws[0] != draws[2] and all(0 <= t < config["vocab"] for t in draws[2])
