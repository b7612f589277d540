"""The gated-linear-attention mixer: a float state matrix per head and sequence instead of cached
keys and values.

    q = Wq h / sqrt(dk),  k = Wk h  ([H, dk]);   v = Wv h  ([H, dv])
    a = sigmoid(W2 (W1 h) + b)^(1/tau)                        one decay per key channel
    S_t = diag(a_t) S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t    per head, S starts at zero
    out = Wo ( concat_h(RMSNorm(o_h) * w) * silu(Wg h) )      w: one vector of dv for all heads

The state is the cache's fixed-size region of the sequence's slot ([H, dk, dv] floats, zeroed when the
slot is handed out); every step continues from it, whatever it was cut into.  The five products
that read h are one matrix (rows q, k, v, g, W1).
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache import CacheNeed, StateNeed
from ..errors import WeightError
from ..registry import register_part
from .base import Mixer, ParamSpec

_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "norm": "norm", "decay_down": "a1", "decay_up": "a2",
          "decay_bias": "a2.b"}


class GatedLinearAttentionMixer(Mixer):
    can_store = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.H, self.dk, self.dv = spec.num_heads, spec.key_dim, spec.value_dim
        self.n = dict(_NAMES)
        self.n.update(dict(getattr(spec, "names", ()) or ()))

    def param_specs(self):
        s, n, H = self.spec, self.n, self.H
        R = s.decay_rank if s.decay_rank else -1          # unless the configuration says it, the tensor does
        return {
            n["q"]: ParamSpec((H * self.dk, s.hidden_size)),
            n["k"]: ParamSpec((H * self.dk, s.hidden_size)),
            n["v"]: ParamSpec((H * self.dv, s.hidden_size)),
            n["gate"]: ParamSpec((H * self.dv, s.hidden_size)),
            n["out"]: ParamSpec((s.hidden_size, H * self.dv)),
            n["norm"]: ParamSpec((self.dv,), role="vector", init="ones_noise"),
            n["decay_down"]: ParamSpec((R, s.hidden_size)),
            n["decay_up"]: ParamSpec((H * self.dk, R)),
            n["decay_bias"]: ParamSpec((H * self.dk,), role="vector", init="wide"),
        }

    def load(self, t):
        n = self.n
        if t[n["decay_down"]].shape[0] != t[n["decay_up"]].shape[1]:
            raise WeightError(f"{n['decay_down']} has {t[n['decay_down']].shape[0]} rows but {n['decay_up']} "
                              f"has {t[n['decay_up']].shape[1]} columns")
        self.w_in = torch.cat([t[n["q"]], t[n["k"]], t[n["v"]], t[n["gate"]], t[n["decay_down"]]], dim=0).contiguous()
        self.w_decay = t[n["decay_up"]].contiguous()
        self.decay_bias = t[n["decay_bias"]].contiguous()
        self.norm = t[n["norm"]].contiguous()
        self.w_out = t[n["out"]].contiguous()

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_decay, self.w_out))

    def cache_need(self):
        return CacheNeed(state=StateNeed((self.H, self.dk, self.dv), torch.float32))

    def forward(self, h, residual, batch, cache, accumulate=True):
        s, ws, T, H, dk, dv = self.spec, self.rt.workspace, h.shape[0], self.H, self.dk, self.dv
        f32 = torch.float32
        proj = ws.take((T, self.w_in.shape[0]), f32)
        ops.gemm(h, self.w_in, proj, ops.EPI_STORE_F32, scratch=ws.take)
        k_off, v_off, g_off, a_off = H * dk, 2 * H * dk, 2 * H * dk + H * dv, 2 * H * dk + 2 * H * dv
        decay = ws.take((T, H * dk), f32)
        ops.gla_decay(proj[:, a_off:], self.w_decay, self.decay_bias, s.decay_tau, decay)
        o = ws.take((T, H * dv), f32)
        ops.gla_scan(proj, 0, k_off, v_off, decay, cache.state, batch.seq_slot, batch.seq_start, o, batch.n_seqs, H, dk, dv,
                     dk ** -0.5)
        y = ws.take((T, H * dv), h.dtype)
        ops.gla_output(o, self.norm, s.norm_eps, proj[:, g_off:], y, H, dv)
        ops.gemm(y, self.w_out, residual, ops.EPI_RESIDUAL if accumulate else ops.EPI_STORE_F32, scratch=ws.take)


register_part("mixer", "gla", GatedLinearAttentionMixer)
