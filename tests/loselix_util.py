"""Test material for the Loselix design: small configurations that differ in every size and option, and a
model-folder writer that is independent of the product's."""

from __future__ import annotations

import json
from pathlib import Path

import torch


def twin(heads, kv, dim, vdim, rot=None, base=10000.0, softcap=20.0, diff=0.3, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "diff": diff,
         "scale": scale if scale is not None else dim ** -0.5}
    if softcap:
        m["softcap"] = softcap
    if rot:
        m["rot"] = {"base": base, "dims": rot}
    return {"type": "attention", "mixer": m}


def soft(heads, kv, dim, vdim, rot=None, base=10000.0, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
    return {"type": "attention_2", "mixer": m}


def sig(heads, kv, dim, coef=0.3, every=16, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale if scale is not None else dim ** -0.5}
    if every:
        m["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention_3", "mixer": m}


def layer(mixer: dict, ff: int | None) -> dict:
    return {**mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(vocab, width, layers, eps=1e-5, loop=None):
    c = {"architecture": "Loselix", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}}
    if loop is not None:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


# sizes in steps of 16 (the tensor-core kernels in bfloat16: the plain one for the softmax mixer with equal sizes,
# the per-size one for the others), three and four query heads a key head, the last two layers run twice
LA = config(200, 64, [layer(soft(4, 1, 32, 32, rot=16), 48),
                      layer(sig(6, 2, 16, coef=0.4, every=8), 80),
                      layer(twin(3, 1, 16, 32, rot=8, softcap=5.0, diff=0.25), 48)], eps=1e-6, loop=(1, 3, 2))
# nothing a multiple of 16 (the CUDA-core kernel in both precisions), as many key heads as query heads, a layer
# without a feed-forward, whole heads rotated, values smaller and larger than keys, no loop at all
LB = config(131, 72, [layer(twin(3, 3, 24, 40, rot=6, base=2e4, softcap=30.0, diff=0.4), 56),
                      layer(sig(6, 2, 20, coef=0.5, every=16), None),
                      layer(soft(2, 1, 24, 8, rot=24, base=500.0), 100)], eps=3e-6)
# heads of 128 (the tcgen05 kernels for the softmax mixer, and for whole tiles of the sigmoid mixer), eight query heads
# on two key heads, a loop over the first two layers that runs three times before the third layer, no query
# temperature, no rotation in the twin layer
LC = config(320, 128, [layer(soft(8, 2, 128, 128, rot=64, base=5e5), 192),
                       layer(sig(4, 2, 128, every=0), 128),
                       layer(twin(4, 2, 64, 64, softcap=0.0, diff=0.1), 64)], eps=1e-5, loop=(0, 2, 3))
# one layer, one head, values of a size of its own: sizes of one
LD = config(90, 40, [layer(soft(1, 1, 16, 24, rot=2), 8)], eps=1e-5, loop=(0, 1, 1))
# keys of 48 with values of 96 and keys of 96 on the tensor cores, a loop in the middle of five layers
LE = config(256, 96, [layer(soft(2, 2, 48, 96, rot=12), 64),
                      layer(twin(4, 2, 48, 96, rot=48, softcap=50.0, diff=0.3), 64),
                      layer(sig(2, 1, 96, coef=0.2, every=32), 64),
                      layer(soft(4, 2, 64, 64, rot=32), None),
                      layer(sig(4, 2, 32, coef=0.3, every=5), 32)], eps=1e-6, loop=(1, 4, 2))
CONFIGS = {"la": LA, "lb": LB, "lc": LC, "ld": LD, "le": LE}
PAGE = {"la": 16, "lb": 8, "lc": 16, "ld": 4, "le": 32}


def tensor_shapes(c: dict) -> dict:
    W, V = c["width"], c["vocab"]
    shapes = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, ly in enumerate(c["layers"]):
        p, mx, kind = f"l{i}", ly["mixer"], ly["type"]
        H, G, D, E = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
        maps = 2 if kind == "attention" else 1
        shapes.update({f"{p}.norm1": (W,), f"{p}.mix.q": (H * maps * D, W), f"{p}.mix.k": (G * maps * D, W),
                       f"{p}.mix.o": (W, H * E)})
        if kind != "attention_3":
            shapes[f"{p}.mix.v"] = (G * E, W)
        if kind == "attention":
            shapes.update({f"{p}.mix.{n}": (D,) for n in ("lq1", "lk1", "lq2", "lk2")})
        if kind == "attention_2":
            shapes[f"{p}.mix.g"] = (H, W)
        if kind == "attention_3":
            shapes.update({f"{p}.mix.g": (H * E, W), f"{p}.mix.q.norm": (H * D,), f"{p}.mix.k.norm": (G * D,),
                           f"{p}.mix.pb": (H,)})
        if ly["mlp"] is not None:
            shapes.update({f"{p}.mlp.up": (ly["mlp"]["ff"], W), f"{p}.mlp.down": (W, ly["mlp"]["ff"])})
    return shapes


def make_weights(c: dict, seed: int) -> dict:
    """Random float32 weights: matrices N(0, 1.5/sqrt(fan_in)) (attention far from uniform), the embedding N(0, 1),
    norm weights 1 + N(0, 0.1), score biases N(-2, 0.5) (sigmoid weights well below one), the vectors that make
    the twin maps' factor N(0, 0.3)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(c).items():
        z = torch.randn(shape, generator=g, dtype=torch.float32)
        if name.endswith(".pb"):
            out[name] = -2.0 + 0.5 * z
        elif name.rsplit(".", 1)[-1] in ("lq1", "lk1", "lq2", "lk2"):
            out[name] = 0.3 * z
        elif len(shape) == 1:
            out[name] = 1.0 + 0.1 * z
        elif name == "embed":
            out[name] = z
        else:
            out[name] = (1.5 / shape[1] ** 0.5) * z
    return out


def stored(weights: dict) -> dict:
    """The values that the folder holds (bfloat16), as float64: both sides compute from the same numbers."""
    return {k: v.to(torch.bfloat16).to(torch.float64) for k, v in weights.items()}


def write_folder(folder, c: dict, weights: dict, dtype=torch.bfloat16) -> Path:
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(c))
    save_file({k: v.to(dtype).contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return folder
