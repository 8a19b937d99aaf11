"""Loselix: config.json -> typed configuration -> `ModelSpec`.

A decoder-only design whose layers are listed one by one in config.json (`layers`: each entry has `type`, the
mixer's sizes under `mixer`, and `mlp` or null).  What the design fixes is fixed here; every size and constant
that config.json carries is read from it.  With u = norm1(x) (RMSNorm, eps = `norm.eps`):

    x <- x + (mixer(u) + ff(u))                     one norm a layer, both branches read it

and `loop` = {start, stop, times} makes layers start .. stop-1 run `times` times in a row with the same weights
(each pass keeps keys and values of its own); before every pass but the first the embedding output is added to
the stream.  The mixers are causal grouped-query attentions:

    "attention"     two score maps a head on the same values (`diff`), scores capped by tanh (`softcap`),
                    rotation of the first `rot.dims` elements of each map
    "attention_2"   softmax attention, rotation of the first `rot.dims` elements, one sigmoid gate a head
    "attention_3"   RMSNorm over the whole query and key projections, values = keys as projected, a query
                    temperature (`q_temp`), sigmoid weights with a bias per head, a sigmoid gate per element

and the feed-forward is down(relu(up(u))^2).  Tensor names: `embed`, `l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`,
`final.norm`, `head`.
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass
from pathlib import Path

from ..config.model_spec import (DenseMLPSpec, GeneralAttentionSpec, LayerSpec, ModelSpec, NormSpec, RopeSpec,
                                 TwinMapsSpec)

ARCHITECTURE = "Loselix"
MIXERS = ("attention", "attention_2", "attention_3")


def _need(d: dict, keys, where: str) -> None:
    missing = [k for k in keys if k not in d]
    if missing:
        raise KeyError(f"config.json: {where} lacks {missing}")


@dataclass(frozen=True)
class LoselixConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple                 # the entries of config.json's `layers`, as read
    loop: tuple | None            # (start, stop, times), or None: every layer runs once

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, c: dict) -> "LoselixConfig":
        _need(c, ("vocab", "width", "layers", "norm"), "the top level")
        _need(c["norm"], ("eps",), "norm")
        loop = c.get("loop")
        if loop is not None:
            _need(loop, ("start", "stop", "times"), "loop")
            loop = (int(loop["start"]), int(loop["stop"]), int(loop["times"]))
        cfg = cls(vocab=int(c["vocab"]), width=int(c["width"]), norm_eps=float(c["norm"]["eps"]),
                  layers=tuple(copy.deepcopy(layer) for layer in c["layers"]), loop=loop)
        cfg.validate()
        return cfg

    @classmethod
    def from_path(cls, path) -> "LoselixConfig":
        p = Path(path)
        if p.is_dir():
            p = p / "config.json"
        return cls.from_dict(json.loads(p.read_text()))

    def validate(self) -> None:
        if self.vocab < 1 or self.width < 1 or not self.layers:
            raise ValueError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ValueError("norm.eps must be positive")
        if self.loop is not None:
            a, b, times = self.loop
            if not 0 <= a < b <= len(self.layers) or times < 1:
                raise ValueError(f"loop {self.loop} does not fit {len(self.layers)} layers")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            kind = layer["type"]
            if kind not in MIXERS:
                raise ValueError(f"{where}: mixer type {kind!r} is not part of this design ({MIXERS})")
            mx = layer["mixer"]
            _need(mx, ("heads", "kv_heads", "dim", "vdim", "scale"), f"{where}.mixer")
            for k in ("heads", "kv_heads", "dim", "vdim"):
                if int(mx[k]) < 1:
                    raise ValueError(f"{where}: mixer.{k} must be positive")
            if int(mx["heads"]) % int(mx["kv_heads"]):
                raise ValueError(f"{where}: heads must be a multiple of kv_heads")
            rot = mx.get("rot")
            if rot is not None:
                _need(rot, ("base", "dims"), f"{where}.mixer.rot")
                if int(rot["dims"]) % 2 or not 2 <= int(rot["dims"]) <= int(mx["dim"]):
                    raise ValueError(f"{where}: rot.dims must be even, positive and at most dim")
            if kind == "attention":
                _need(mx, ("diff",), f"{where}.mixer")
            if kind == "attention_3":
                if int(mx["vdim"]) != int(mx["dim"]):
                    raise ValueError(f"{where}: the values are the keys, so vdim must equal dim")
                qt = mx.get("q_temp")
                if qt is not None:
                    _need(qt, ("coef", "every"), f"{where}.mixer.q_temp")
                    if int(qt["every"]) < 1:
                        raise ValueError(f"{where}: q_temp.every must be positive")
            ml = layer.get("mlp")
            if ml is not None:
                _need(ml, ("kind", "ff"), f"{where}.mlp")
                if ml["kind"] != "dense":
                    raise ValueError(f"{where}: feed-forward kind {ml['kind']!r} is not part of this design")
                if int(ml["ff"]) < 1:
                    raise ValueError(f"{where}: mlp.ff must be positive")

    def to_dict(self) -> dict:
        """config.json content for this configuration."""
        d = {"architecture": ARCHITECTURE, "layers": [copy.deepcopy(layer) for layer in self.layers],
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.loop is not None:
            d["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        return d

    # ----------------------------------------------------------------- the model
    def run_order(self) -> tuple:
        """(the order in which the layers run, the places right before which the embedding is added again)."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n)), ()
        a, b, times = self.loop
        order, again = list(range(a)), []
        for t in range(times):
            if t > 0:
                again.append(len(order))
            order += range(a, b)
        return tuple(order + list(range(b, n))), tuple(again)

    def _mixer(self, kind: str, mx: dict) -> GeneralAttentionSpec:
        eps, W = self.norm_eps, self.width
        rot = mx.get("rot")
        common = dict(hidden_size=W, num_heads=int(mx["heads"]), num_kv_heads=int(mx["kv_heads"]),
                      key_dim=int(mx["dim"]), value_dim=int(mx["vdim"]), scale=float(mx["scale"]), prefix="mix",
                      score_cap=float(mx["softcap"]) if mx.get("softcap") else None,
                      position=None if rot is None else
                      RopeSpec(dim=int(rot["dims"]), theta=float(rot["base"]), exact_table=True))
        if kind == "attention":
            return GeneralAttentionSpec(**common, twin=TwinMapsSpec(offset=float(mx["diff"]), eps=eps))
        if kind == "attention_2":
            return GeneralAttentionSpec(**common, gate="head")
        qt = mx.get("q_temp")
        return GeneralAttentionSpec(**common, whole_norm_eps=eps, values_from_keys=True, weights="sigmoid",
                                    score_bias=True, gate="element",
                                    query_temperature=None if qt is None else (float(qt["coef"]), int(qt["every"])))

    def to_spec(self) -> ModelSpec:
        eps, W = self.norm_eps, self.width
        layers = []
        for i, layer in enumerate(self.layers):
            ml = layer.get("mlp")
            ff = None if ml is None else DenseMLPSpec(hidden_size=W, intermediate_size=int(ml["ff"]),
                                                      activation="relu2", prefix="mlp")
            layers.append(LayerSpec(prefix=f"l{i}", mixer=self._mixer(layer["type"], layer["mixer"]), feed_forward=ff,
                                    mixer_norm=NormSpec(W, eps, "norm1"), ffn_norm=None, kind="parallel"))
        order, again = self.run_order()
        spec = ModelSpec(architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=W, layers=tuple(layers),
                         final_norm=NormSpec(W, eps, "final.norm"), embedding_name="embed", lm_head_name="head",
                         schedule=order, reinject=again)
        spec.validate()
        return spec
