"""Test material for the Guronex design: small configurations that differ in every size and option, and a
model-folder writer that is independent of the product's."""

from __future__ import annotations

import json
from pathlib import Path

import torch


def mixer(heads, dim, rot_dim, vdim, kv_rank, base=10000.0, scale=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "rot": {"base": base, "dims": rot_dim}, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def moe(experts, top, ff, groups=None):
    rt = {"experts": experts, "top": top}
    if groups is not None:
        rt["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": rt}


def layer(mx, ml):
    return {"type": "latent_attention", "mixer": mx, "mlp": ml}


def config(vocab, width, layers, eps=1e-5, mult=0.5, side=None):
    c = {"architecture": "Guronex", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
         "residual_mult": mult}
    if side is not None:
        c["token_side"] = {"dim": side}
    return c


# cache rows of 64 (the mma.sync attention in bfloat16); a reader of layer 0 with other heads; a layer without a
# feed-forward; groups that restrict the choice
GA = config(200, 64, [layer(mixer(2, 16, 16, 16, 48), moe(8, 2, 32, (4, 2))),
                      layer(mixer(4, 8, 16, 24, 48, kv_from=0), moe(8, 2, 32, (4, 2))),
                      layer(mixer(2, 16, 16, 16, 48, base=500.0), None)], eps=1e-6, mult=0.5, side=8)
# rows of 48 and 96 (the CUDA-core attention in both precisions), two cache groups, an odd vocabulary, top 1 with
# one group, and groups of which all are kept; no token input
GB = config(301, 96, [layer(mixer(3, 24, 8, 20, 40, base=2e4), moe(6, 1, 40, (1, 1))),
                      layer(mixer(5, 16, 24, 16, 72), moe(12, 3, 24, (3, 3)))], eps=3e-6, mult=1.0)
# rows of 128 with eight heads (the tcgen05 attention in bfloat16), readers of two different layers, experts
# without groups, a token input of 12 columns
GC = config(320, 128, [layer(mixer(8, 32, 16, 48, 112), moe(16, 4, 48, (2, 1))),
                       layer(mixer(8, 32, 16, 48, 112, base=1e6), moe(16, 4, 48)),
                       layer(mixer(8, 32, 16, 48, 112, kv_from=0), moe(16, 4, 48, (4, 3))),
                       layer(mixer(4, 64, 16, 32, 112, base=1e6, kv_from=1), moe(16, 4, 48, (2, 1)))],
            eps=1e-5, mult=0.25, side=12)
# more than 16 heads on one cache row, more than 32 experts, a width that is no multiple of 16
GD = config(150, 80, [layer(mixer(20, 8, 8, 8, 24), moe(40, 5, 16, (5, 2)))], eps=1e-5, mult=0.7, side=5)
# a long cache row (384) with values of 320
GE = config(128, 64, [layer(mixer(2, 32, 64, 32, 320), moe(4, 2, 32))], eps=1e-5, mult=0.4, side=4)
# experts of 128 and more (the grouped tcgen05 product in bfloat16), one size no multiple of its tiles
GF = config(256, 128, [layer(mixer(4, 16, 16, 32, 48), moe(8, 2, 128, (2, 1))),
                       layer(mixer(4, 16, 16, 32, 48, kv_from=0), moe(8, 3, 136))], eps=1e-5, mult=0.5, side=8)
# 24 heads on a cache row of 128: the tcgen05 attention takes them as two groups of 12
GG = config(180, 96, [layer(mixer(24, 8, 48, 8, 80), moe(4, 2, 16))], eps=1e-5, mult=0.6)
# nothing a multiple of 8: width 100, vocabulary 131, a cache row of 22, three heads of 10+4 with values of 14, five
# experts of 12, a token input of 3 columns
GH = config(131, 100, [layer(mixer(3, 10, 4, 14, 18), moe(5, 2, 12)),
                       layer(mixer(2, 6, 4, 10, 18, kv_from=0), None)], eps=2e-6, mult=0.8, side=3)
CONFIGS = {"ga": GA, "gb": GB, "gc": GC, "gd": GD, "ge": GE, "gf": GF, "gg": GG, "gh": GH}
PAGE = {"ga": 16, "gb": 8, "gc": 16, "gd": 4, "ge": 32, "gf": 16, "gg": 16, "gh": 16}


def tensor_shapes(c: dict) -> dict:
    W, V, L = c["width"], c["vocab"], len(c["layers"])
    side = c.get("token_side")
    shapes = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    if side is not None:
        shapes["side.embed"] = (V, L * side["dim"])
    for i, ly in enumerate(c["layers"]):
        p, mx = f"l{i}", ly["mixer"]
        H = mx["heads"]
        shapes.update({f"{p}.norm1": (W,), f"{p}.mix.q": (H * (mx["dim"] + mx["rot_dim"]), W),
                       f"{p}.mix.uk": (H * mx["dim"], mx["kv_rank"]), f"{p}.mix.uv": (H * mx["vdim"], mx["kv_rank"]),
                       f"{p}.mix.g": (H * mx["vdim"], W), f"{p}.mix.o": (W, H * mx["vdim"])})
        if mx.get("kv_from") is None:
            shapes[f"{p}.mix.dkv"] = (mx["kv_rank"] + mx["rot_dim"], W)
            shapes[f"{p}.mix.dkv.norm"] = (mx["kv_rank"],)
        if ly["mlp"] is not None:
            shapes[f"{p}.norm2"] = (W,)
            shapes[f"{p}.mlp.router"] = (ly["mlp"]["router"]["experts"], W)
            for e in range(ly["mlp"]["router"]["experts"]):
                shapes[f"{p}.mlp.e{e}.up"] = (ly["mlp"]["expert"]["ff"], W)
                shapes[f"{p}.mlp.e{e}.down"] = (W, ly["mlp"]["expert"]["ff"])
        if side is not None:
            shapes.update({f"{p}.side.gate": (side["dim"], W), f"{p}.side.proj": (W, side["dim"]),
                           f"{p}.side.norm": (W,)})
    return shapes


def make_weights(c: dict, seed: int) -> dict:
    """Random float32 weights: matrices N(0, 1.5/sqrt(fan_in)) (attention far from uniform, router scores far from
    equal), tables N(0, 1), norm weights 1 + N(0, 0.1)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(c).items():
        z = torch.randn(shape, generator=g, dtype=torch.float32)
        if len(shape) == 1:
            out[name] = 1.0 + 0.1 * z
        elif name in ("embed", "side.embed"):
            out[name] = z
        else:
            out[name] = (1.5 / shape[1] ** 0.5) * z
    return out


def write_folder(folder, c: dict, weights: dict, dtype=torch.bfloat16) -> Path:
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(c))
    save_file({k: v.to(dtype).contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return folder
