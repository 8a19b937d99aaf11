"""Plain, slow, whole-sequence implementation of the Guronex design (on the CPU, float64 or
float32): the oracle that the engine is compared with.

No cache, no batching, no kernels: one function per mechanism, each written from the
design's equations.  It shares no code with the product package: it reads config.json
keys and safetensors names itself.

The design, in this file's notation (h: a layer's input, [tokens, width]; m: the residual
multiplier; rms(y) = y / sqrt(mean(y^2) + eps)):

    x0          = embed[token]
    x          <- x + m * rms(mixer(x)) * norm1
    x          <- x + m * rms(ff(x)) * norm2                (if the layer has a feed-forward)
    x          <- x + m * rms(side(x, token)) * side.norm   (if the model has per-layer token inputs)
    logits      = head (rms(x) * final.norm)

mixer = latent attention: queries per head [dim | rot_dim]; keys are made from a latent
c = rms(first kv_rank rows of W_dkv h) * dkv.norm and one rotated part of rot_dim shared by all
heads; key_h = [W_uk_h c | rot(k_r)], value_h = W_uv_h c; causal softmax; heads gated by
sigmoid(W_g h); W_o.  A layer with `kv_from` = j takes c and rot(k_r) from layer j.

ff = routed experts: s = softmax(W_router h) over all experts; experts in `count` groups of
neighbours; a group scores as its best expert; only experts of the `keep` best groups may be
chosen; the `top` best of those are chosen; out = sum s_e * W_down_e gelu(W_up_e h).
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
    """y divided by its root mean square, eps inside the root."""
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def rms_norm(y, weight, eps):
    return unit_rms(y, eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def rotate(u: torch.Tensor, positions: torch.Tensor, base: float) -> torch.Tensor:
    """u [..., tokens, dims]: element i is paired with i + dims/2; the pair (a, b) at position p
    becomes (a cos t - b sin t, b cos t + a sin t), t = p * base^(-2i/dims)."""
    dims = u.shape[-1]
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(torch.float64)[:, None] * freq[None, :]
    cos, sin = torch.cos(ang).to(u.dtype), torch.sin(ang).to(u.dtype)
    a, b = u[..., :half], u[..., half:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)


# ------------------------------------------------------------------ latent attention
def latent_and_rotated_key(h, w, prefix, mx, eps, positions):
    """What a layer with a W_dkv of its own leaves for itself and for the layers that read it:
    c [tokens, kv_rank] and the rotated key part [tokens, rot_dim]."""
    r = mx["kv_rank"]
    d = h @ w[f"{prefix}.dkv"].T
    c = rms_norm(d[:, :r], w[f"{prefix}.dkv.norm"], eps)
    kr = rotate(d[:, r:], positions, mx["rot"]["base"])
    return c, kr


def latent_attention(h, w, prefix, mx, eps, positions, shared):
    """`shared` = (c, rotated key part) of the layer this one reads, or None."""
    T = h.shape[0]
    H, dn, dr, dv = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"]
    assert mx["rot"]["dims"] == dr
    c, kr = shared if shared is not None else latent_and_rotated_key(h, w, prefix, mx, eps, positions)
    q = (h @ w[f"{prefix}.q"].T).reshape(T, H, dn + dr)
    qn = q[:, :, :dn]
    qr = rotate(q[:, :, dn:].transpose(0, 1), positions, mx["rot"]["base"]).transpose(0, 1)
    kn = (c @ w[f"{prefix}.uk"].T).reshape(T, H, dn)
    v = (c @ w[f"{prefix}.uv"].T).reshape(T, H, dv)
    scores = (torch.einsum("thd,shd->hts", qn, kn) + torch.einsum("thd,sd->hts", qr, kr)) * mx["scale"]
    visible = torch.arange(T)[None, :] <= torch.arange(T)[:, None]          # [query, key]
    scores = scores.masked_fill(~visible[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    o = torch.einsum("hts,shd->thd", p, v).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ w[f"{prefix}.g"].T)
    return o @ w[f"{prefix}.o"].T, (c, kr)


# -------------------------------------------------------------------- routed experts
def route(h, w_router, rt):
    """(chosen [tokens, top] expert indices, their weights): softmax over all experts, the best `keep`
    groups by their best expert, the `top` best experts inside those; weights are the scores as they are."""
    E, top = rt["experts"], rt["top"]
    s = torch.softmax((h @ w_router.T).to(torch.float64), dim=-1)
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = rt.get("groups")
    if groups is not None:
        n, keep = groups["count"], groups["keep"]
        best = s.reshape(-1, n, E // n).max(dim=-1).values                   # [tokens, groups]
        kept = best.topk(keep, dim=-1).indices
        gmask = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
        allowed = gmask[:, :, None].expand(-1, n, E // n).reshape(-1, E)
    chosen = s.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
    return chosen, s.gather(1, chosen).to(h.dtype)


def route_margin(h, w_router, rt):
    """Per token, how far the choice is from going another way: the smallest difference of router logits
    between something that was taken (the last chosen expert, the last kept group) and the best that was not.
    A 16-bit computation may choose otherwise where this is small; such a token's result is then another."""
    E, top = rt["experts"], rt["top"]
    z = (h @ w_router.T).to(torch.float64)
    chosen, _ = route(h, w_router, rt)
    taken = torch.zeros_like(z, dtype=torch.bool).scatter_(1, chosen, True)
    margin = torch.full((h.shape[0],), float("inf"), dtype=torch.float64)
    allowed = torch.ones_like(taken)
    groups = rt.get("groups")
    if groups is not None and groups["keep"] < groups["count"]:
        n, keep = groups["count"], groups["keep"]
        best = z.reshape(-1, n, E // n).max(dim=-1).values.sort(dim=-1, descending=True).values
        margin = best[:, keep - 1] - best[:, keep]
        kept = z.reshape(-1, n, E // n).max(dim=-1).values >= best[:, keep - 1:keep]
        allowed = kept[:, :, None].expand(-1, n, E // n).reshape(-1, E)
    rest = z.masked_fill(taken | ~allowed, float("-inf")).max(dim=-1).values
    last = z.masked_fill(~taken, float("inf")).min(dim=-1).values
    return torch.minimum(margin, last - rest)


def routed_experts(h, w, prefix, ml, forced=None):
    """`forced` [tokens, top]: these experts are taken instead of the router's choice (their weights are still the
    router's scores): for following a 16-bit computation whose choice went the other way at a close call."""
    chosen, weight = route(h, w[f"{prefix}.router"], ml["router"])
    if forced is not None:
        chosen = forced
        weight = torch.softmax((h @ w[f"{prefix}.router"].T).to(torch.float64), dim=-1).gather(1, chosen).to(h.dtype)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            a = gelu_erf(h[t] @ w[f"{prefix}.e{e}.up"].T)
            out[t] += g * (a @ w[f"{prefix}.e{e}.down"].T)
    return out


# ------------------------------------------------------------- per-layer token input
def token_side(x, tokens, w, layer, i, dim, eps):
    e = w["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    g = gelu_tanh(x @ w[f"{layer}.side.gate"].T) * e
    return rms_norm(g @ w[f"{layer}.side.proj"].T, w[f"{layer}.side.norm"], eps)


# -------------------------------------------------------------------------- the model
def forward(cfg: dict, w: dict, tokens, return_layers: bool = False, margins: list | None = None,
            forced: list | None = None, free: list | None = None, round_inputs=None):
    """Logits [tokens, vocab] for one whole sequence (and the stream after every layer).  `margins`, if given,
    receives one tensor per routed layer: every token's `route_margin` there; `free` the router's own choice
    there; `forced` (one [tokens, top] tensor per routed layer) makes the layers take those experts;
    `round_inputs` (a function) is applied to what every branch reads: with a rounding to 16 bits it shows how
    far rounding alone moves the logits of a position."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    side = cfg.get("token_side")
    x = w["embed"][tokens]
    kept = {}
    after = []
    routed = 0
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        if layer["type"] != "latent_attention":
            raise ValueError(f"layer {i}: mixer {layer['type']!r}")
        mx = layer["mixer"]
        src = mx.get("kv_from")
        rd = round_inputs if round_inputs is not None else (lambda t: t)
        y, mine = latent_attention(rd(x), w, f"{p}.mix", mx, eps, positions, kept[src] if src is not None else None)
        if src is None:
            kept[i] = mine
        x = x + m * rms_norm(y, w[f"{p}.norm1"], eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "moe":
                raise ValueError(f"layer {i}: feed-forward {layer['mlp']['kind']!r}")
            if margins is not None:
                margins.append(route_margin(rd(x), w[f"{p}.mlp.router"], layer["mlp"]["router"]))
            if free is not None:
                free.append(route(rd(x), w[f"{p}.mlp.router"], layer["mlp"]["router"])[0])
            force = forced[routed] if forced is not None else None
            routed += 1
            x = x + m * rms_norm(routed_experts(rd(x), w, f"{p}.mlp", layer["mlp"], force), w[f"{p}.norm2"], eps)
        if side is not None:
            x = x + m * token_side(rd(x), tokens, w, p, i, side["dim"], eps)
        after.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(after)) if return_layers else logits
