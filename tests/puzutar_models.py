"""Small Puzutar configurations with random weights for the tests, written as model folders.

P differs from layer to layer in every size the design has (heads, head sizes, latent size, window, rotated
share, feed-forward or none) and has two blocks that read another block's latent rows with windows of their own.
T has the sizes that the tensor-core attention kernel takes, U sizes that fit no kernel's pieces.  Q has one norm group, no side input, no window, a head count that no kernel tile divides and a latent wider than
128.  R keeps three sizes equal to one (a head count, a head size, the side input's width), norm groups of four
values, and two blocks on one latent whose windows end one before and on a page border.
"""
from __future__ import annotations

import json
import os

import numpy as np


def mixer(heads, dim, rot_dim, vdim, kv_rank, window, scale=None, rot_dims=None, base=10000.0, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank,
             scale=float(scale if scale is not None else (dim + rot_dim) ** -0.5), rot=dict(base=base, dims=rot_dim if rot_dims is None else rot_dims))
    if window:
        m["mask"] = dict(size=window)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def layer(m, ff):
    return dict(type="latent_attention", mixer=m, mlp=dict(kind="dense", ff=ff) if ff else None)


CONFIG_P = dict(architecture="Puzutar", vocab=160, width=96, norm=dict(eps=1e-5, groups=3), token_side=dict(dim=8), layers=[
    layer(mixer(2, 16, 8, 24, 40, 20, rot_dims=4), 136),
    layer(mixer(3, 8, 8, 12, 40, 33, rot_dims=4, kv_from=0), 64),
    layer(mixer(5, 8, 12, 16, 24, 9, base=500.0), 0),
    layer(mixer(1, 24, 12, 8, 24, 5, base=500.0, kv_from=2), 200),
    layer(mixer(2, 4, 12, 8, 24, 17, base=500.0, kv_from=2), 72),
])
CONFIG_Q = dict(architecture="Puzutar", vocab=300, width=64, norm=dict(eps=1e-6, groups=1), layers=[
    layer(mixer(5, 16, 32, 20, 160, 0, base=1e6), 96),
    layer(mixer(6, 32, 32, 8, 160, 40, base=1e6, kv_from=0), 96),
])
CONFIG_R = dict(architecture="Puzutar", vocab=64, width=48, norm=dict(eps=1e-5, groups=12), token_side=dict(dim=1), layers=[
    layer(mixer(1, 1, 2, 1, 16, 16, scale=1.5), 48),
    layer(mixer(4, 12, 4, 12, 8, 31, scale=0.7), 48),
    layer(mixer(4, 12, 4, 12, 8, 32, scale=0.7, kv_from=1), 48),
])
# Shapes that the bfloat16 engine's tensor-core attention takes (latents of 32, 64 and 96 values, rotated parts of 16 and 32): fewer
# heads than a row tile, more than one (two head groups), a reader with a window of its own, and one block without a window.
CONFIG_T = dict(architecture="Puzutar", vocab=200, width=128, norm=dict(eps=1e-5, groups=4), token_side=dict(dim=16), layers=[
    layer(mixer(12, 16, 16, 16, 64, 40), 256),
    layer(mixer(3, 8, 16, 24, 64, 70, kv_from=0), 128),
    layer(mixer(20, 8, 32, 8, 96, 0, base=1e5), 128),
    layer(mixer(2, 32, 16, 32, 32, 33), 0),
])
# Sizes that fit no kernel's pieces: a width that is no multiple of 8, five norm groups, seven heads, rotated parts of 8 of which 6
# turn, a window of one position (a token sees itself only) beside one wider than any prompt, a side input three values wide, and a
# latent the tensor-core path takes (512 values) behind 64 rotated ones.
CONFIG_U = dict(architecture="Puzutar", vocab=97, width=100, norm=dict(eps=1e-4, groups=5), token_side=dict(dim=3), layers=[
    layer(mixer(7, 24, 8, 40, 72, 1, rot_dims=6, base=77.0), 50),
    layer(mixer(2, 10, 8, 6, 72, 1000, rot_dims=6, base=77.0, kv_from=0), 0),
    layer(mixer(1, 16, 64, 32, 512, 45, base=1e6), 60),
])
CONFIGS = {"P": (CONFIG_P, 11), "Q": (CONFIG_Q, 12), "R": (CONFIG_R, 13), "T": (CONFIG_T, 14), "U": (CONFIG_U, 15)}


def to_bf16_values(a):
    """Rounds to values that bfloat16 holds, so that the file, the engine in either type and the plain model agree."""
    from liyab_b200.weights import bf16_to_f32, f32_to_bf16
    return bf16_to_f32(f32_to_bf16(np.asarray(a, dtype=np.float32)))


def random_weights(config, seed):
    rng = np.random.default_rng(seed)
    V, W, L = config["vocab"], config["width"], len(config["layers"])
    out = {}

    def mat(name, rows, cols, std=None):
        out[name] = rng.normal(0.0, std if std is not None else cols ** -0.5, size=(rows, cols))

    def vec(name, n, mean, std):
        out[name] = rng.normal(mean, std, size=n)

    mat("embed", V, W, 1.0)
    side = config.get("token_side")
    if side:
        mat("side.embed", V, L * side["dim"], 1.0)
    for i, l in enumerate(config["layers"]):
        m = l["mixer"]
        H, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        vec(f"l{i}.norm1", W, 1.0, 0.2)
        mat(f"l{i}.mix.q", H * (dim + rot), W)
        if "kv_from" not in m:
            mat(f"l{i}.mix.dkv", rank + rot, W)
            vec(f"l{i}.mix.dkv.norm", rank, 1.0, 0.2)
        mat(f"l{i}.mix.uk", H * dim, rank)
        mat(f"l{i}.mix.uv", H * vdim, rank)
        mat(f"l{i}.mix.o", W, H * vdim)
        if l["mlp"]:
            ff = l["mlp"]["ff"]
            mat(f"l{i}.mlp.up", ff, W)
            vec(f"l{i}.mlp.up.b", ff, 0.0, 0.3)
            mat(f"l{i}.mlp.down", W, ff)
            vec(f"l{i}.mlp.down.b", W, 0.0, 0.3)
            vec(f"l{i}.mlp.act", 2, 0.3, 0.6)
        out[f"l{i}.shift"] = rng.uniform(0.0, 1.0, size=W)
        if side:
            mat(f"l{i}.side.gate", side["dim"], W)
            mat(f"l{i}.side.proj", W, side["dim"], 1.0)
            vec(f"l{i}.side.norm", W, 0.5, 0.2)
    vec("final.norm", W, 1.0, 0.2)
    return {k: to_bf16_values(v) for k, v in out.items()}


def write_model(folder, config, weights):
    from liyab_b200.weights import f32_to_bf16, write_safetensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {k: f32_to_bf16(v) for k, v in weights.items()},
                      tags={k: "BF16" for k in weights})
    return folder


def model_folder(base, name):
    config, seed = CONFIGS[name]
    weights = random_weights(config, seed)
    return write_model(os.path.join(base, f"puzutar_{name}"), config, weights), config, weights
