"""Small Vosurax configurations with random weights for the tests, written as model folders.

A differs from layer to layer in every size the design has, rotates part of a head, has a block without a feed-forward,
experts with and without a shared one, and a stretch of two blocks that runs three times.  B has the sizes the bfloat16
engine's tensor-core kernels take and a stretch that starts at the first block.  C has sizes that fit no kernel's pieces:
a width that is no multiple of 8, value heads wider than one tile of the memory's state, a chunk of one position beside one
wider than any prompt and a branch without a mask, every expert chosen (top = experts), and a stretch that runs once.
D keeps sizes equal to one (heads, key/value heads, one expert, a value head of one value).
"""
from __future__ import annotations

import json
import os

import numpy as np


def retention(heads, dim, vdim, decay, rot_dims, base=10000.0):
    return dict(heads=heads, dim=dim, vdim=vdim, decay=[float(d) for d in decay], rot=dict(base=base, dims=rot_dims))


def side_by_side(heads, kv_heads, dim, vdim, scale, chunk, r_heads, r_dim, r_vdim, cap):
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=float(scale))
    if chunk:
        left["mask"] = dict(size=chunk)
    return dict(left=left, right=dict(heads=r_heads, dim=r_dim, vdim=r_vdim, gate_cap=float(cap)))


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, shared=0):
    m = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
    if shared:
        m["shared"] = dict(ff=shared)
    return m


def layer(mixer, mlp):
    return dict(type="parallel" if "left" in mixer else "retention", mixer=mixer, mlp=mlp)


CONFIG_A = dict(architecture="Vosurax", vocab=160, width=96, norm=dict(eps=1e-5), loop=dict(start=1, stop=3, times=3), layers=[
    layer(retention(3, 16, 24, [0.9, 0.97, 0.995], 8, 500.0), dense(136)),
    layer(side_by_side(4, 2, 12, 20, 0.3, 20, 2, 8, 24, 10.0), moe(6, 2, 24, 40)),
    layer(side_by_side(3, 3, 16, 8, 0.25, 33, 5, 12, 8, 15.0), None),
    layer(retention(1, 32, 16, [0.98], 32), moe(4, 1, 16)),
])
CONFIG_B = dict(architecture="Vosurax", vocab=200, width=128, norm=dict(eps=1e-6), loop=dict(start=0, stop=2, times=2), layers=[
    layer(side_by_side(4, 2, 64, 64, 0.125, 32, 2, 32, 64, 9.0), moe(8, 2, 64, 64)),
    layer(retention(2, 32, 64, [0.95, 0.9975], 16, 5e5), dense(256)),
    layer(side_by_side(8, 2, 32, 32, 0.18, 48, 4, 16, 32, 8.0), dense(128)),
])
CONFIG_C = dict(architecture="Vosurax", vocab=97, width=100, norm=dict(eps=1e-4), loop=dict(start=2, stop=3, times=1), layers=[
    layer(side_by_side(6, 1, 24, 40, 0.2, 1, 3, 10, 70, 6.0), moe(3, 3, 20, 12)),
    layer(side_by_side(2, 2, 10, 6, 0.4, 1000, 1, 20, 130, 20.0), dense(50)),
    layer(side_by_side(5, 5, 8, 8, 0.35, 0, 2, 6, 10, 13.0), None),
    layer(retention(2, 10, 70, [0.5, 1.0], 6, 77.0), moe(5, 2, 8, 0)),
])
CONFIG_D = dict(architecture="Vosurax", vocab=64, width=48, norm=dict(eps=1e-5), layers=[
    layer(retention(1, 2, 1, [0.9], 2, 10.0), moe(1, 1, 8, 8)),
    layer(side_by_side(1, 1, 1, 1, 1.0, 16, 1, 1, 1, 1.0), dense(1)),
    layer(side_by_side(2, 1, 16, 16, 0.25, 31, 1, 16, 16, 11.0), dense(48)),
])
CONFIGS = {"A": (CONFIG_A, 21), "B": (CONFIG_B, 22), "C": (CONFIG_C, 23), "D": (CONFIG_D, 24)}


def to_bf16_values(a):
    """Rounds to values that bfloat16 holds, so that the file, the engine in either type and the plain model agree."""
    from liyab_b200.weights import bf16_to_f32, f32_to_bf16
    return bf16_to_f32(f32_to_bf16(np.asarray(a, dtype=np.float32)))


def random_weights(config, seed, router_std=3.0):
    rng = np.random.default_rng(seed)
    V, W = config["vocab"], config["width"]
    out = {}

    def mat(name, rows, cols, std=None):
        out[name] = rng.normal(0.0, std if std is not None else cols ** -0.5, size=(rows, cols))

    def vec(name, n, mean, std):
        out[name] = rng.normal(mean, std, size=n)

    def memory(p, m, gated):
        H, D, E = m["heads"], m["dim"], m["vdim"]
        mat(p + "q", H * D, W)
        mat(p + "k", H * D, W)
        mat(p + "v", H * E, W)
        mat(p + "g", H * E, W)
        mat(p + "o", W, H * E)
        if gated:
            mat(p + "i", H, W)
            mat(p + "f", H, W)
            vec(p + "i.b", H, 0.0, 1.0)
            vec(p + "f.b", H, 2.0, 1.0)
            vec(p + "norm", H * E, 1.0, 0.2)

    mat("embed", V, W, 1.0)
    mat("head", V, W)
    vec("final.norm", W, 0.0, 0.2)
    loop = config.get("loop")
    if loop and loop["stop"] > loop["start"]:
        out["loop.step"] = rng.normal(0.0, 0.5, size=(loop["times"], W))
    for i, l in enumerate(config["layers"]):
        p = f"l{i}."
        vec(p + "norm1", W, 0.0, 0.2)
        m = l["mixer"]
        if l["type"] == "retention":
            memory(p + "mix.", m, False)
        else:
            a = m["left"]
            H, G, D, E = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            q = p + "mix.left."
            mat(q + "q", H * D, W)
            mat(q + "k", G * D, W)
            mat(q + "v", G * E, W)
            mat(q + "g", H * E, W)
            mat(q + "o", W, H * E)
            vec(q + "q.b", H * D, 0.0, 0.3)
            vec(q + "k.b", G * D, 0.0, 0.3)
            vec(q + "v.b", G * E, 0.0, 0.3)
            vec(q + "q.norm", D, 1.0, 0.2)
            vec(q + "k.norm", D, 1.0, 0.2)
            memory(p + "mix.right.", m["right"], True)
            vec(p + "mix.left.out", W, 1.0, 0.2)
            vec(p + "mix.right.out", W, 1.0, 0.2)
        mlp = l["mlp"]
        if mlp:
            vec(p + "norm2", W, 0.0, 0.2)
            if mlp["kind"] == "dense":
                mat(p + "mlp.up", mlp["ff"], W)
                mat(p + "mlp.down", W, mlp["ff"])
            else:
                F = mlp["expert"]["ff"]
                mat(p + "mlp.router", mlp["router"]["experts"], W, router_std * W ** -0.5)
                for e in range(mlp["router"]["experts"]):
                    mat(f"{p}mlp.e{e}.gate", F, W)
                    mat(f"{p}mlp.e{e}.up", F, W)
                    mat(f"{p}mlp.e{e}.down", W, F)
                if mlp.get("shared"):
                    S = mlp["shared"]["ff"]
                    mat(p + "mlp.shared.gate", S, W)
                    mat(p + "mlp.shared.up", S, W)
                    mat(p + "mlp.shared.down", W, S)
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
    return write_model(os.path.join(base, f"vosurax_{name}"), config, weights), config, weights
