"""The latent-attention mixer: keys and values of all heads are products of one small cached
vector per token, and the kernels never build them.

With h the mixer's input, H heads, per head dn unrotated and dr rotated query/key channels, values
of dv, and a latent of rk:

    cq = RMSNorm(Dq h) * w_q;   q = Uq cq -> per head [a_h (dn) | b_h (dr)]       (no q latent: q = Uq h)
    [c' | r'] = Dkv h;   c = RMSNorm(c') * w_kv;   r = rotate(r'), one for all heads
    k_h = [Uk_h c | r],  v_h = Uv_h c,   score = (a_h . Uk_h c + rotate(b_h) . r) * scale
    softmax over the window's keys, with exp(sink_h) added to the denominator
    out = O ( concat_h(sum_j p_j v_hj) * sigmoid(G h) )

Only [c | r] is cached (one plane, one "head" of rk + dr numbers per token).  Scores are taken as
(Uk_h^T a_h) . c_j + rotate(b_h) . r_j and values as Uv_h (sum_j p_j c_j): one product per head
before and one after the attention, which then runs over the latent alone.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache import CacheNeed, KVNeed
from ..errors import ConfigError
from ..registry import build_part, register_part
from .base import Mixer, ParamSpec

_NAMES = {"q_down": "dq", "q_norm": "dq.norm", "q_up": "uq", "kv_down": "dkv", "kv_norm": "dkv.norm", "k_up": "uk",
          "v_up": "uv", "sink": "sink", "gate": "g", "out": "o"}


class LatentAttentionMixer(Mixer):
    can_store = True

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.H, self.dn, self.dr, self.dv, self.rk = spec.num_heads, spec.nope_dim, spec.rope_dim, spec.v_dim, spec.kv_rank
        if self.dr > 0 and spec.position is None:
            raise ConfigError("latent attention with rotated channels needs a position encoding")
        self.position = build_part("position", spec.position, rt=rt) if spec.position is not None else None
        if self.position is not None and self.position.rotary_dim != self.dr:
            raise ConfigError(f"the rotated width ({self.position.rotary_dim}) must equal the rotated channels per head ({self.dr})")
        self.n = dict(_NAMES)
        self.n.update(dict(getattr(spec, "names", ()) or ()))

    def param_specs(self):
        s, n, H = self.spec, self.n, self.H
        p = {
            n["q_up"]: ParamSpec((H * (self.dn + self.dr), s.q_rank or s.hidden_size)),
            n["kv_down"]: ParamSpec((self.rk + self.dr, s.hidden_size)),
            n["kv_norm"]: ParamSpec((self.rk,), role="vector", init="ones_noise"),
            n["k_up"]: ParamSpec((H * self.dn, self.rk)),
            n["v_up"]: ParamSpec((H * self.dv, self.rk)),
            n["out"]: ParamSpec((s.hidden_size, H * self.dv)),
        }
        if s.q_rank:
            p[n["q_down"]] = ParamSpec((s.q_rank, s.hidden_size))
            p[n["q_norm"]] = ParamSpec((s.q_rank,), role="vector", init="ones_noise")
        if s.sink:
            p[n["sink"]] = ParamSpec((H,), role="vector", init="wide")
        if s.gate:
            p[n["gate"]] = ParamSpec((H * self.dv, s.hidden_size))
        return p

    def load(self, t):
        s, n, H = self.spec, self.n, self.H
        self.w_qup = t[n["q_up"]].contiguous()
        self.w_qdown = t[n["q_down"]].contiguous() if s.q_rank else None
        self.q_norm = t[n["q_norm"]].contiguous() if s.q_rank else None
        # the latent's product and the gate's read the same input: one matrix, rows [c' | r' | gate]
        self.w_kvg = torch.cat([t[n["kv_down"]]] + ([t[n["gate"]]] if s.gate else []), dim=0).contiguous()
        self.kv_norm = t[n["kv_norm"]].contiguous()
        self.w_kup = t[n["k_up"]].view(H, self.dn, self.rk).transpose(1, 2).contiguous()      # [h][latent][channel]: Uk_h^T
        self.w_vup = t[n["v_up"]].view(H, self.dv, self.rk).contiguous()                      # [h][value][latent]: Uv_h
        self.sink = t[n["sink"]].contiguous() if s.sink else None
        self.w_out = t[n["out"]].contiguous()

    def weight_bytes(self):
        ws = [self.w_qup, self.w_qdown, self.w_kvg, self.w_kup, self.w_vup, self.w_out]
        return sum(w.numel() * w.element_size() for w in ws if w is not None)

    def cache_need(self):
        return CacheNeed(kv=KVNeed(1, self.rk + self.dr, self.spec.window, planes=1))

    def forward(self, h, residual, batch, cache, accumulate=True):
        s, ws, T, H = self.spec, self.rt.workspace, h.shape[0], self.H
        dn, dr, dv, rk = self.dn, self.dr, self.dv, self.rk
        f32 = torch.float32
        if s.q_rank:
            cqf = ws.take((T, s.q_rank), f32)
            ops.gemm(h, self.w_qdown, cqf, ops.EPI_STORE_F32, scratch=ws.take)
            cq = ws.take((T, s.q_rank), h.dtype)
            ops.rmsnorm(cqf, self.q_norm, cq, s.norm_eps)
        else:
            cq = h
        q = ws.take((T, H * (dn + dr)), f32)
        ops.gemm(cq, self.w_qup, q, ops.EPI_STORE_F32, scratch=ws.take)
        kvg = ws.take((T, self.w_kvg.shape[0]), f32)
        ops.gemm(h, self.w_kvg, kvg, ops.EPI_STORE_F32, scratch=ws.take)
        pages, pos = batch.pages[cache.kv_group], self.position
        freq = pos.freq if pos is not None else self.kv_norm      # unread when nothing is rotated
        mscale = pos.mscale if pos is not None else 1.0
        if cache.writes_kv:
            ops.latent_kv_store(kvg, self.kv_norm, s.norm_eps, freq, mscale, rk, dr, batch.tok_seq, batch.tok_pos, pages,
                                cache.k, cache.page_size)
        qa = ws.take((T, H * (rk + dr)), f32)
        ops.headwise_gemm(q, dn + dr, self.w_kup, qa, rk + dr, scale=s.scale)
        if dr:
            ops.rotate_heads(q, dn + dr, dn, qa, rk + dr, rk, freq, mscale, batch.tok_pos, H, dr, scale=s.scale)
        lat = ws.take((T, H * rk), f32)
        ops.latent_attention(qa, lat, cache.k, self.sink, batch.tok_seq, batch.tok_pos, pages, H, rk, dr, cache.page_size,
                             s.window, batch=batch, scratch=ws.take)
        att = ws.take((T, H * dv), h.dtype)
        ops.headwise_gemm(lat, rk, self.w_vup, att, dv, gate=kvg[:, rk + dr:] if s.gate else None)
        ops.gemm(att, self.w_out, residual, ops.EPI_RESIDUAL if accumulate else ops.EPI_STORE_F32, scratch=ws.take)


register_part("mixer", "latent_attention", LatentAttentionMixer)
