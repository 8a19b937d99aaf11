"""Guronex: config.json -> typed configuration -> `ModelSpec`.

A decoder-only design whose layers are listed one by one in config.json (`layers`: each
entry has `type`, the mixer's sizes under `mixer`, and `mlp` or null).  What the design
fixes is fixed here; every size and constant that config.json carries is read from it:

    x <- x + m * norm1(mixer(x));  x <- x + m * norm2(ff(x));  x <- x + m * side_norm(side(x, token))

with m = `residual_mult`, RMSNorm (eps = `norm.eps`) on each branch's OUTPUT, the mixer a
latent attention (queries [dim | rot_dim] per head, a normed latent of `kv_rank` and one
rotated key part shared by the heads in the cache, a sigmoid output gate; `kv_from` = j
makes a layer read layer j's cache), the feed-forward a mixture of experts with
softmax scores, group-limited choice and un-renormalised weights, and `token_side.dim`
columns of a shared per-token table as a further branch after the feed-forward.
Tensor names: `embed`, `side.embed`, `l<i>.norm1|norm2`, `l<i>.mix.*`, `l<i>.mlp.*`,
`l<i>.side.*`, `final.norm`, `head`.
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass
from pathlib import Path

from ..config.model_spec import (LatentAttentionSpec, LayerSpec, ModelSpec, NormSpec, RopeSpec, RoutedExpertsSpec,
                                 TokenInputSpec)

ARCHITECTURE = "Guronex"
MIXERS = ("latent_attention",)


def _need(d: dict, keys, where: str) -> None:
    missing = [k for k in keys if k not in d]
    if missing:
        raise KeyError(f"config.json: {where} lacks {missing}")


@dataclass(frozen=True)
class GuronexConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    side_dim: int | None          # columns of the per-token table that a layer takes; None: no such branch
    layers: tuple                 # the entries of config.json's `layers`, as read

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, c: dict) -> "GuronexConfig":
        _need(c, ("vocab", "width", "layers", "norm", "residual_mult"), "the top level")
        _need(c["norm"], ("eps",), "norm")
        side = c.get("token_side")
        if side is not None:
            _need(side, ("dim",), "token_side")
        cfg = cls(vocab=int(c["vocab"]), width=int(c["width"]), norm_eps=float(c["norm"]["eps"]),
                  residual_mult=float(c["residual_mult"]), side_dim=None if side is None else int(side["dim"]),
                  layers=tuple(copy.deepcopy(layer) for layer in c["layers"]))
        cfg.validate()
        return cfg

    @classmethod
    def from_path(cls, path) -> "GuronexConfig":
        p = Path(path)
        if p.is_dir():
            p = p / "config.json"
        return cls.from_dict(json.loads(p.read_text()))

    def validate(self) -> None:
        if self.vocab < 1 or self.width < 1 or not self.layers:
            raise ValueError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ValueError("norm.eps must be positive")
        if self.side_dim is not None and self.side_dim < 1:
            raise ValueError("token_side.dim must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            if layer["type"] not in MIXERS:
                raise ValueError(f"{where}: mixer type {layer['type']!r} is not part of this design ({MIXERS})")
            mx = layer["mixer"]
            _need(mx, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"), f"{where}.mixer")
            _need(mx["rot"], ("base", "dims"), f"{where}.mixer.rot")
            if int(mx["rot"]["dims"]) != int(mx["rot_dim"]):
                raise ValueError(f"{where}: rot.dims must equal rot_dim (the rotated part is rotated whole)")
            if int(mx["rot_dim"]) % 2 or int(mx["rot_dim"]) < 2:
                raise ValueError(f"{where}: rot_dim must be even and positive")
            for k in ("heads", "dim", "vdim", "kv_rank"):
                if int(mx[k]) < 1:
                    raise ValueError(f"{where}: mixer.{k} must be positive")
            j = mx.get("kv_from")
            if j is not None:
                if not 0 <= int(j) < i:
                    raise ValueError(f"{where}: kv_from={j} must name an earlier layer")
                src = self.layers[int(j)]["mixer"]
                if src.get("kv_from") is not None:
                    raise ValueError(f"{where}: kv_from={j} names a layer without a cache of its own")
                same = ("kv_rank", "rot_dim")
                if any(int(src[k]) != int(mx[k]) for k in same) or \
                        any(float(src["rot"][k]) != float(mx["rot"][k]) for k in ("base", "dims")):
                    raise ValueError(f"{where}: kv_rank, rot_dim and rotation must equal those of layer {j}")
            ml = layer.get("mlp")
            if ml is not None:
                _need(ml, ("kind", "router", "expert"), f"{where}.mlp")
                if ml["kind"] != "moe":
                    raise ValueError(f"{where}: feed-forward kind {ml['kind']!r} is not part of this design")
                rt = ml["router"]
                _need(rt, ("experts", "top"), f"{where}.mlp.router")
                _need(ml["expert"], ("ff",), f"{where}.mlp.expert")
                E, top = int(rt["experts"]), int(rt["top"])
                n, keep = self._groups(rt)
                if E < 1 or not 1 <= top <= E or E % n or not 1 <= keep <= n or top > keep * (E // n):
                    raise ValueError(f"{where}: router sizes do not fit (experts {E}, top {top}, groups {n}, keep {keep})")

    @staticmethod
    def _groups(rt: dict) -> tuple:
        g = rt.get("groups")
        return (1, 1) if g is None else (int(g["count"]), int(g["keep"]))

    def to_dict(self) -> dict:
        """config.json content for this configuration."""
        d = {"architecture": ARCHITECTURE, "layers": [copy.deepcopy(layer) for layer in self.layers],
             "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab,
             "width": self.width}
        if self.side_dim is not None:
            d["token_side"] = {"dim": self.side_dim}
        return d

    # ----------------------------------------------------------------- the model
    def to_spec(self) -> ModelSpec:
        eps, W, L = self.norm_eps, self.width, len(self.layers)
        layers = []
        for i, layer in enumerate(self.layers):
            mx, ml = layer["mixer"], layer.get("mlp")
            mixer = LatentAttentionSpec(
                hidden_size=W, num_heads=int(mx["heads"]), plain_dim=int(mx["dim"]), rot_dim=int(mx["rot_dim"]),
                value_dim=int(mx["vdim"]), latent_dim=int(mx["kv_rank"]), scale=float(mx["scale"]),
                position=RopeSpec(dim=int(mx["rot"]["dims"]), theta=float(mx["rot"]["base"])),
                latent_norm_eps=eps, output_gate=True, prefix="mix")
            ff = None
            if ml is not None:
                n, keep = self._groups(ml["router"])
                ff = RoutedExpertsSpec(hidden_size=W, num_experts=int(ml["router"]["experts"]),
                                       top_k=int(ml["router"]["top"]), expert_size=int(ml["expert"]["ff"]),
                                       n_groups=n, keep_groups=keep, scoring="softmax", renormalize=False,
                                       activation="gelu", prefix="mlp")
            side = None
            if self.side_dim is not None:
                side = TokenInputSpec(hidden_size=W, dim=self.side_dim, offset=i * self.side_dim,
                                      table_name="side.embed", table_width=L * self.side_dim, vocab_size=self.vocab,
                                      eps=eps, prefix="side")
            j = mx.get("kv_from")
            layers.append(LayerSpec(prefix=f"l{i}", mixer=mixer, feed_forward=ff,
                                    mixer_norm=NormSpec(W, eps, "norm1"),
                                    ffn_norm=NormSpec(W, eps, "norm2") if ff is not None else None,
                                    cache_from=None if j is None else int(j), kind="branch_norm",
                                    residual_scale=self.residual_mult, token_input=side))
        spec = ModelSpec(architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=W, layers=tuple(layers),
                         final_norm=NormSpec(W, eps, "final.norm"), embedding_name="embed", lm_head_name="head")
        spec.validate()
        return spec
