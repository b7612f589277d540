"""The routed feed-forward: a router picks `top_k` of the experts for every token.

    s = softmax(R h) over all experts (float);  chosen: the top_k largest s
    out = sum over chosen e of w_e * Down_e act(Up_e h),   w_e = s_e (or s_e / sum of the chosen s)

The experts' matrices are stacked at load time ([E, F, D] and [E, D, F]) so that a kernel finds an
expert by its index; which experts a token uses never reaches the host, so a recorded step replays.
"""

from __future__ import annotations

import torch

from .. import ops
from ..errors import ConfigError
from ..registry import register_part
from .base import FeedForward, ParamSpec


class RoutedFeedForward(FeedForward):
    can_store = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        if spec.activation not in ops.ACTIVATIONS:
            raise ConfigError(f"unknown activation {spec.activation!r}: {', '.join(ops.ACTIVATIONS)}")
        self.act = ops.ACTIVATIONS[spec.activation]

    def _names(self, e):
        return tuple(n.format(e=e) for n in self.spec.expert_names)

    def param_specs(self):
        s = self.spec
        p = {s.router_name: ParamSpec((s.num_experts, s.hidden_size), init="wide")}
        for e in range(s.num_experts):
            up, down = self._names(e)
            p[up] = ParamSpec((s.expert_size, s.hidden_size))
            p[down] = ParamSpec((s.hidden_size, s.expert_size))
        return p

    def load(self, t):
        s = self.spec
        self.router = t[s.router_name].contiguous()
        self.up = torch.stack([t[self._names(e)[0]] for e in range(s.num_experts)]).contiguous()
        self.down = torch.stack([t[self._names(e)[1]] for e in range(s.num_experts)]).contiguous()

    def weight_bytes(self):
        """What a step of one token reads: the router and top_k experts."""
        s = self.spec
        per = 2 * s.expert_size * s.hidden_size * self.up.element_size()
        return self.router.numel() * self.router.element_size() + s.top_k * per

    def forward(self, h, residual, batch, accumulate=True):
        s, ws, T = self.spec, self.rt.workspace, h.shape[0]
        ids = ws.take((T, s.top_k), torch.int32)
        weights = ws.take((T, s.top_k), torch.float32)
        ops.moe_route(h, self.router, ids, weights, s.top_k, s.renormalize)
        if ops.moe_grouped_ok(h, self.up):
            ops.moe_experts_grouped(h, self.up, self.down, ids, weights, residual, self.act, accumulate, ws.take)
            return
        mid = ws.take((T * s.top_k, s.expert_size), h.dtype)
        ops.moe_experts(h, self.up, self.down, ids, weights, mid, residual, self.act, accumulate)


register_part("ffn", "moe", RoutedFeedForward)
