"""The dense gated feed-forward: down( act(gate(h)) * up(h) ), added to the residual stream
(crates/backends/backend_common/src/generic_mlp.rs:83-96; silu(x) = x / (1 + exp(-x)),
kernels.rs:677-687).  act is silu unless the spec names another (gelu in its tanh or erf form); the
product's fused epilogue serves silu, the others take the product and then the activation kernel.

gate_proj and up_proj are one matrix here.  When the intermediate size is a multiple of 8
their rows alternate in groups of 8 (8 gate rows, the 8 up rows of the same channels, ...), so
that a kernel holding 16 consecutive output columns has both halves of 8 channels; otherwise
the up rows follow all gate rows.
"""

from __future__ import annotations

import torch

from .. import ops
from ..errors import ConfigError
from ..registry import register_part
from .base import FeedForward, ParamSpec

INTERLEAVE = 8


def join_gate_up(gate: torch.Tensor, up: torch.Tensor):
    inter, hidden = gate.shape
    if inter % INTERLEAVE == 0:
        g = gate.view(inter // INTERLEAVE, INTERLEAVE, hidden)
        u = up.view(inter // INTERLEAVE, INTERLEAVE, hidden)
        return torch.cat([g, u], dim=1).reshape(2 * inter, hidden).contiguous(), INTERLEAVE
    return torch.cat([gate, up], dim=0).contiguous(), 0


class SwiGLU(FeedForward):
    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.wgu = self.wd = None
        self.interleave = 0
        self.names = tuple(getattr(spec, "names", ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
        act = getattr(spec, "activation", "silu")
        if act not in ops.ACTIVATIONS:
            raise ConfigError(f"unknown activation {act!r}: {', '.join(ops.ACTIVATIONS)}")
        self.act = ops.ACTIVATIONS[act]

    def param_specs(self):
        s, (gate, up, down) = self.spec, self.names
        return {
            gate: ParamSpec((s.intermediate_size, s.hidden_size)),
            up: ParamSpec((s.intermediate_size, s.hidden_size)),
            down: ParamSpec((s.hidden_size, s.intermediate_size)),
        }

    def load(self, tensors):
        gate, up, down = self.names
        self.wgu, self.interleave = join_gate_up(tensors[gate], tensors[up])
        self.wd = tensors[down].contiguous()

    def weight_bytes(self):
        return (self.wgu.numel() + self.wd.numel()) * self.wgu.element_size()

    shares_norms = True
    can_store = True

    def forward(self, h, residual, batch, next_norm=None, accumulate=True):
        ws, T, inter = self.rt.workspace, h.shape[0], self.spec.intermediate_size
        act = ws.take((T, inter), self.rt.dtype)
        if self.act == ops.ACT_SILU:
            ops.gemm_swiglu(h, self.wgu, act, self.interleave, ws.take)
        else:
            gu = ws.take((T, 2 * inter), self.rt.dtype)
            ops.gemm(h, self.wgu, gu, scratch=ws.take)
            ops.swiglu(gu, act, self.interleave, self.act)
        if not accumulate:
            return ops.gemm(act, self.wd, residual, ops.EPI_STORE_F32, scratch=ws.take)
        return ops.gemm(act, self.wd, residual, ops.EPI_RESIDUAL, next_norm=next_norm, scratch=ws.take)


register_part("ffn", "swiglu", SwiGLU)
