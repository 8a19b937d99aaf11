"""A branch fed by the token id: e = this layer's columns of a shared per-token table,

    branch = proj( gelu_tanh(gate(x)) * e )

(the products through `ops.linear`, the gate with the table lookup in csrc/token_input.cu).  The block norms the
branch with this part's own RMSNorm weight.  Every layer that has such a branch names the same table tensor.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, TensorSpec
from .registry import register_token_input


class TokenInput(Part):
    kernels = ("token_input", "gemm_simt")

    def __init__(self, spec, prefix, ctx):
        self.spec, self.ctx = spec, ctx
        self.prefix = f"{prefix}.{spec.prefix}" if spec.prefix else prefix
        self.eps = float(spec.eps)
        self.table = self.w_gate = self.w_proj = self.norm_weight = None

    def tensor_specs(self):
        p, s = self.prefix, self.spec
        return {s.table_name: TensorSpec((s.vocab_size, s.table_width)),
                f"{p}.gate": TensorSpec((s.dim, s.hidden_size)),
                f"{p}.proj": TensorSpec((s.hidden_size, s.dim)),
                f"{p}.norm": TensorSpec((s.hidden_size,), kind="vector", init="ones_normal")}

    def bind(self, tensors):
        p, s = self.prefix, self.spec
        self.table = tensors[s.table_name]
        if not self.table.is_contiguous():
            raise ValueError(f"{s.table_name} must be contiguous")
        self.w_gate = self.compute_weight(tensors[f"{p}.gate"], self.ctx).contiguous()
        self.w_proj = self.compute_weight(tensors[f"{p}.proj"], self.ctx).contiguous()
        self.norm_weight = tensors[f"{p}.norm"].contiguous()

    def forward(self, x, step):
        dt = self.ctx.dtype
        z = ops.linear(x, self.w_gate, torch.float32)        # kept in 32-bit for the activation
        g = ops.token_gate(z, step.token_ids, self.table, self.spec.offset, out_dtype=dt)
        return ops.linear(g, self.w_proj, dt, parts_ok=True)


register_token_input("token_input", TokenInput)
