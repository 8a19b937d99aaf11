"""Plain, slow, whole-sequence implementation of the Loselix design (on the CPU, float64 or
float32): the oracle that the engine is compared with.

No cache, no batching, no kernels: one function per mechanism, each written from the
design's equations.  It shares no code with the product package: it reads config.json
keys and safetensors names itself.

The design in this file's notation (x: the stream [tokens, width]; rms(y) = y / sqrt(mean(y^2) + eps)):

    e           = embed[token]                                  x starts as e
    layer:   u  = rms(x) * norm1;   x <- x + mixer(u) + ff(u)   (one norm, two readers, one sum)
    loop:       layers start .. stop-1 run `times` times with the same weights (every pass has its own
                keys and values); before every pass but the first, x <- x + e
    logits      = head (rms(x) * final.norm)

mixers, all causal, H query heads on G key/value heads (query head h reads head h // (H/G)):

    soft_gated  (type "attention_2")  rotated q, k; softmax(q.k * scale); head h times sigmoid(g_h . u)
    sigmoid     (type "attention_3")  q, k normed over the whole projection; v = k before its norm; q times
                                      a temperature that grows with the position; weights
                                      sigmoid(q.k * scale + pb_h), not normalised; times sigmoid(W_g u)
    twin        (type "attention")    two score maps per head on the same values, scores capped by tanh;
                                      o = a1 - lam * a2, then rms(o) * (1 - diff)

ff = W_down relu(W_up u)^2.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def read_config(folder) -> dict:
    return json.loads((Path(folder) / "config.json").read_text())


def read_weights(folder, dtype=torch.float64) -> dict:
    from safetensors import safe_open

    out = {}
    for shard in sorted(Path(folder).glob("*.safetensors")):
        with safe_open(str(shard), framework="pt") as f:
            for key in f.keys():
                t = f.get_tensor(key)
                out[key] = t.to(dtype) if t.is_floating_point() else t
    return out


# ----------------------------------------------------------------------- small parts
def unit_rms(y: torch.Tensor, eps: float) -> torch.Tensor:
    """y divided by its root mean square over the last axis, eps inside the root."""
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def rms_norm(y, weight, eps):
    return unit_rms(y, eps) * weight


def rotate_first(y: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """y [tokens, heads, size]: element i < dims/2 of every head is paired with element i + dims/2 and the pair is
    turned by the angle position * base^(-2i/dims); elements from `dims` on stay."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = float(base) ** (-2.0 * i / dims)
    ang = positions.to(torch.float64)[:, None] * freq[None, :]
    c, s = torch.cos(ang).to(y.dtype)[:, None, :], torch.sin(ang).to(y.dtype)[:, None, :]
    a, b = y[..., :half], y[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, y[..., dims:]], dim=-1)


def causal_scores(q: torch.Tensor, k: torch.Tensor, scale: float) -> torch.Tensor:
    """q [T, H, D], k [T, G, D] -> scores [H, T, T] (query, key), query head h on key head h // (H/G)."""
    H, G = q.shape[1], k.shape[1]
    kk = k.repeat_interleave(H // G, dim=1)
    return torch.einsum("ihd,jhd->hij", q, kk) * scale


def visible(T: int) -> torch.Tensor:
    i = torch.arange(T)
    return i[None, :] <= i[:, None]


def softmax_attend(scores: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """scores [H, T, T], v [T, G, E] -> [T, H, E]: softmax over the visible keys."""
    H, T, _ = scores.shape
    vv = v.repeat_interleave(H // v.shape[1], dim=1)
    s = scores.masked_fill(~visible(T)[None], -math.inf)
    return torch.einsum("hij,jhe->ihe", torch.softmax(s, dim=-1), vv)


def sigmoid_attend(scores: torch.Tensor, bias: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Weights sigmoid(score + bias_h) on the visible keys, zero elsewhere; no normalisation over keys."""
    H, T, _ = scores.shape
    vv = v.repeat_interleave(H // v.shape[1], dim=1)
    w = torch.sigmoid(scores + bias[:, None, None]) * visible(T)[None].to(scores.dtype)
    return torch.einsum("hij,jhe->ihe", w, vv)


def tanh_cap(s: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(s / cap)


def query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    """1 + coef * ln(floor((p + 1) / every) + 1) for every position p."""
    steps = torch.div(positions.to(torch.int64) + 1, int(every), rounding_mode="floor")
    return 1.0 + coef * torch.log(steps.to(torch.float64) + 1.0)


# --------------------------------------------------------------------------- mixers
def mixer_soft_gated(u, pos, w, p, mx, eps):
    T = u.shape[0]
    H, G, D, E = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (u @ w[f"{p}.q"].T).view(T, H, D)
    k = (u @ w[f"{p}.k"].T).view(T, G, D)
    v = (u @ w[f"{p}.v"].T).view(T, G, E)
    rot = mx.get("rot")
    if rot is not None:
        q, k = rotate_first(q, pos, rot["dims"], rot["base"]), rotate_first(k, pos, rot["dims"], rot["base"])
    o = softmax_attend(causal_scores(q, k, mx["scale"]), v)
    gate = torch.sigmoid(u @ w[f"{p}.g"].T)                 # [T, H]: one number a head
    return (o * gate[:, :, None]).reshape(T, H * E) @ w[f"{p}.o"].T


def mixer_sigmoid(u, pos, w, p, mx, eps):
    T = u.shape[0]
    H, G, D = mx["heads"], mx["kv_heads"], mx["dim"]
    q_all, k_all = u @ w[f"{p}.q"].T, u @ w[f"{p}.k"].T
    v = k_all.view(T, G, D)                                 # the values are the keys as projected
    q = rms_norm(q_all, w[f"{p}.q.norm"], eps).view(T, H, D)
    k = rms_norm(k_all, w[f"{p}.k.norm"], eps).view(T, G, D)
    qt = mx.get("q_temp")
    if qt is not None:
        q = q * query_temperature(pos, qt["coef"], qt["every"]).to(q.dtype)[:, None, None]
    o = sigmoid_attend(causal_scores(q, k, mx["scale"]), w[f"{p}.pb"].to(q.dtype), v)
    gate = torch.sigmoid(u @ w[f"{p}.g"].T)                 # [T, H * D]: element by element
    return (o.reshape(T, H * D) * gate) @ w[f"{p}.o"].T


def twin_lambda(w, p, diff: float) -> float:
    a = float((w[f"{p}.lq1"].double() * w[f"{p}.lk1"].double()).sum())
    b = float((w[f"{p}.lq2"].double() * w[f"{p}.lk2"].double()).sum())
    return math.exp(a) - math.exp(b) + diff


def mixer_twin(u, pos, w, p, mx, eps):
    T = u.shape[0]
    H, G, D, E = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (u @ w[f"{p}.q"].T).view(T, H * 2, D)               # head by head: [map 1, map 2]
    k = (u @ w[f"{p}.k"].T).view(T, G * 2, D)
    v = (u @ w[f"{p}.v"].T).view(T, G, E)
    rot = mx.get("rot")
    if rot is not None:
        q, k = rotate_first(q, pos, rot["dims"], rot["base"]), rotate_first(k, pos, rot["dims"], rot["base"])
    q, k = q.view(T, H, 2, D), k.view(T, G, 2, D)
    maps = []
    for m in range(2):
        s = causal_scores(q[:, :, m], k[:, :, m], mx["scale"])
        if mx.get("softcap"):
            s = tanh_cap(s, mx["softcap"])
        maps.append(softmax_attend(s, v))
    diff = mx["diff"]
    o = maps[0] - twin_lambda(w, p, diff) * maps[1]
    o = unit_rms(o, eps) * (1.0 - diff)                     # over the head's values, no weight
    return o.reshape(T, H * E) @ w[f"{p}.o"].T


MIXERS = {"attention": mixer_twin, "attention_2": mixer_soft_gated, "attention_3": mixer_sigmoid}


def feed_forward(u, w, p):
    return torch.relu(u @ w[f"{p}.up"].T) ** 2 @ w[f"{p}.down"].T


# ---------------------------------------------------------------------------- model
def run_order(cfg: dict) -> list:
    """[(layer, whether the embedding output is added before it)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for t in range(times):
        order += [(i, t > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(cfg: dict, w: dict, tokens, return_layers: bool = False):
    """Logits [T, vocab] for one sequence from position 0 (and the stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(tokens.numel())
    e = w["embed"][tokens]
    x = e.clone()
    streams = []
    for i, add_e in run_order(cfg):
        ly, p = cfg["layers"][i], f"l{i}"
        if add_e:
            x = x + e
        u = rms_norm(x, w[f"{p}.norm1"], eps)
        branch = MIXERS[ly["type"]](u, pos, w, f"{p}.mix", ly["mixer"], eps)
        if ly.get("mlp") is not None:
            branch = branch + feed_forward(u, w, f"{p}.mlp")
        x = x + branch
        streams.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(streams)) if return_layers else logits
