"""Arrangement of a layer: pre-norm with two residual sums
(jllm/model/common.py:140-147),

    h = h + mixer(norm1(h));  h = h + feed_forward(norm2(h)).

The stream `h` is float32 in every mode.  A block hands back its last branch output as
`delta`, not yet added, so that the next norm (of the next block, or the final one) adds
and normalises in one pass over the stream.  A branch output is a tensor [n, hidden] or an
`ops.PartialSum` (the parts of a product whose k was cut); the norms take either.
"""

from __future__ import annotations

import torch

from .. import ops
from ..ops import trace_range
from .base import Part
from .registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, TOKEN_INPUTS, build, register_block


class PreNormBlock(Part):
    def __init__(self, spec, prefix, ctx):
        p = spec.prefix
        self.spec = spec
        self.mixer_norm = build(NORMS, "norm", spec.mixer_norm, p, ctx)
        self.mixer = build(MIXERS, "mixer", spec.mixer, p, ctx)
        self.ffn_norm = build(NORMS, "norm", spec.ffn_norm, p, ctx)
        self.feed_forward = build(FEED_FORWARDS, "feed-forward", spec.feed_forward, p, ctx)
        if spec.cache_from is not None:
            if not hasattr(self.mixer, "writes_cache"):
                raise ValueError(f"{p}: this mixer cannot read another layer's cache")
            self.mixer.writes_cache = False

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)

    def tensor_specs(self):
        out = {}
        for part in self.parts():
            out.update(part.tensor_specs())
        return out

    def bind(self, tensors):
        for part in self.parts():
            part.bind(tensors)

    def forward(self, h, delta, step, cache):
        step.stream_copy = None
        with trace_range("mixer_norm"):
            x = self.mixer_norm.norm(h, delta)
        with trace_range("mixer"):
            a = self.mixer.forward(x, step, cache)
        with trace_range("ffn_norm"):
            x = self.ffn_norm.norm(h, a)
        with trace_range("feed_forward"):
            return h, self.feed_forward.forward(x, step)


register_block("pre_norm", PreNormBlock)


class BranchNormBlock(Part):
    """A layer that norms every branch's OUTPUT before adding it, scaled, to the stream:

        h += m * norm1(mixer(h));  h += m * norm2(feed_forward(h));  h += m * norm_t(token_input(h, token))

    with m = `residual_scale`; the feed-forward and the token input are optional.  The branches read the stream
    itself, rounded to the compute type: each residual update (csrc/branch_norm.cu: norm, scale, sum and the
    rounded copy in one pass, 32-bit) hands the next branch its input.  Nothing is left un-added at the end, so
    the block takes a pending `delta` from an arrangement before it and returns none."""

    kernels = ("branch_norm",)

    def __init__(self, spec, prefix, ctx):
        p = spec.prefix
        self.spec, self.ctx = spec, ctx
        self.scale = float(spec.residual_scale)
        self.mixer_norm = build(NORMS, "norm", spec.mixer_norm, p, ctx)
        self.mixer = build(MIXERS, "mixer", spec.mixer, p, ctx)
        self.feed_forward = self.ffn_norm = self.token_input = None
        if spec.feed_forward is not None:
            self.ffn_norm = build(NORMS, "norm", spec.ffn_norm, p, ctx)
            self.feed_forward = build(FEED_FORWARDS, "feed-forward", spec.feed_forward, p, ctx)
        if spec.token_input is not None:
            self.token_input = build(TOKEN_INPUTS, "token input", spec.token_input, p, ctx)
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and not hasattr(norm, "weight"):
                raise ValueError(f"{p}: this arrangement needs norms with a plain weight")
        if spec.cache_from is not None:
            if not hasattr(self.mixer, "writes_cache"):
                raise ValueError(f"{p}: this mixer cannot read another layer's cache")
            self.mixer.writes_cache = False

    def parts(self):
        return tuple(part for part in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward, self.token_input)
                     if part is not None)

    def tensor_specs(self):
        out = {}
        for part in self.parts():
            out.update(part.tensor_specs())
        return out

    def bind(self, tensors):
        for part in self.parts():
            part.bind(tensors)

    def forward(self, h, delta, step, cache):
        dt = self.ctx.dtype
        # the stream rounded to the compute type, as the block before left it (only a block of this kind does)
        x, step.stream_copy = step.stream_copy, None
        if delta is not None:
            ops.residual_add(h, delta)
            x = None
        if x is None or dt == torch.float32:
            x = ops.cast_rows(h, dt)
        with trace_range("mixer"):
            a = self.mixer.forward(x, step, cache)
        with trace_range("mixer_norm"):
            x = self._add(h, a, self.mixer_norm.weight, self.mixer_norm.eps)
        if self.feed_forward is not None:
            with trace_range("feed_forward"):
                a = self.feed_forward.forward(x, step)
            with trace_range("ffn_norm"):
                x = self._add(h, a, self.ffn_norm.weight, self.ffn_norm.eps)
        if self.token_input is not None:
            with trace_range("token_input"):
                a = self.token_input.forward(x, step)
                x = self._add(h, a, self.token_input.norm_weight, self.token_input.eps)
        step.stream_copy = x if dt != torch.float32 else None
        return h, None

    def _add(self, h, branch, weight, eps):
        """The residual update; returns what the next branch reads (in 32-bit mode the stream itself)."""
        if self.ctx.dtype == torch.float32:
            ops.branch_norm_add(h, branch, weight, eps, self.scale)
            return h
        return ops.branch_norm_add(h, branch, weight, eps, self.scale, x_dtype=self.ctx.dtype)


register_block("branch_norm", BranchNormBlock)


def build_block(spec, ctx):
    return build(BLOCKS, "block", spec, spec.prefix, ctx)
