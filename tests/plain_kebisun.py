"""A plain, slow implementation of the Kebisun decoder: whole sequences, no cache, no batching,
one function per mechanism, written from the design's equations.  It shares no code with the
library: it parses config.json and the safetensors file itself and computes with torch on the CPU.

The design in this file's notation (T tokens, D = width; all positions count from 0):

  x_0 = E[token] * s_e
  a layer:  x <- x + ls1 * LN1(mixer(x));  x <- x + ls2 * LN2(ff(x))    (sublayers read x itself;
            LN(y) = (y - mean) / sqrt(var + eps) * w with the biased variance; a layer may lack ff)
  logits = head LN_final(x)

`dtype` is the dtype of all arithmetic (float64 for a ground truth).  Weights are used as stored
(bfloat16 values widened exactly).  `store`, where given, is applied to every activation that an
engine would keep in its activation dtype between two kernels (`bf16_storage` rounds those to
bfloat16): what the number format alone does to the logits follows from it.
"""

from __future__ import annotations

import json
import math
import struct
from typing import Dict, Sequence

import numpy as np
import torch


# ---- reading a model folder ---------------------------------------------------------------------
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        if info["dtype"] == "BF16":
            u = np.frombuffer(data[b:e], dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).copy())
        elif info["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(data[b:e], dtype="<f4").copy())
        elif info["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(data[b:e], dtype="<i4").copy())
        else:
            raise ValueError(f"dtype {info['dtype']} of {name}")
        out[name] = t.reshape(info["shape"])
    return out


def bf16_storage(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(t.dtype)


def _keep(t):
    return t


# ---- small functions --------------------------------------------------------------------------
def layer_norm(y, w, eps):
    mean = y.mean(-1, keepdim=True)
    var = ((y - mean) ** 2).mean(-1, keepdim=True)
    return (y - mean) / torch.sqrt(var + eps) * w


def rms_norm(y, w, eps):
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def silu(z):
    return z / (1.0 + torch.exp(-z))


# ---- rotation -----------------------------------------------------------------------------------
def rotary_frequencies(rot: dict, dtype):
    """(f [dims/2], m): the pair (i, i + dims/2) turns by p * f_i; cos and sin are multiplied by m.
    f_i = base^(-2i/dims); with `scaling` (factor F, original L, fast, slow):
    d(t) = dims * ln(L / (2 pi t)) / (2 ln base), lo = max(floor(d(fast)), 0),
    hi = min(ceil(d(slow)), dims - 1), r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    f_i <- f_i / F * r_i + f_i * (1 - r_i), m = 0.1 ln F + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    m = 1.0
    sc = rot.get("scaling")
    if sc:
        F, L = float(sc["factor"]), float(sc["original"])

        def d(t):
            return dims * math.log(L / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo = max(math.floor(d(float(sc["fast"]))), 0)
        hi = min(math.ceil(d(float(sc["slow"]))), dims - 1)
        r = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / F * r + f * (1.0 - r)
        m = 0.1 * math.log(F) + 1.0
    return f.to(dtype), m


def rotate(u, positions, f, m):
    """u [..., T, dims]: the pair (u_i, u_{i+dims/2}) at position p becomes
    (u_i cos a - u_{i+h} sin a, u_{i+h} cos a + u_i sin a) with a = p f_i, cos and sin times m."""
    half = u.shape[-1] // 2
    a = positions.to(f.dtype)[:, None] * f[None, :]
    c, s = torch.cos(a) * m, torch.sin(a) * m
    u1, u2 = u[..., :half], u[..., half:]
    return torch.cat([u1 * c - u2 * s, u2 * c + u1 * s], dim=-1)


# ---- mixers -------------------------------------------------------------------------------------
def latent_attention(h, W, m, eps, store=_keep):
    """Windowed softmax attention whose keys and values come out of one small latent per token.
    W: the mixer's tensors by short name; m: the mixer's sizes."""
    T = h.shape[0]
    H, dn, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    f, ms = rotary_frequencies(m["rot"], h.dtype)
    cq = store(rms_norm(h @ W["dq"].T, W["dq.norm"], eps))
    q = (cq @ W["uq"].T).view(T, H, dn + dr)
    q_n, q_r = q[..., :dn], q[..., dn:]
    kv = h @ W["dkv"].T
    c = store(rms_norm(kv[:, :rk], W["dkv.norm"], eps))
    k_r = store(rotate(kv[:, rk:], pos, f, ms))                      # one rotated part for all heads
    q_r = rotate(q_r.transpose(0, 1), pos, f, ms).transpose(0, 1)
    k_n = (c @ W["uk"].T).view(T, H, dn)
    v = (c @ W["uv"].T).view(T, H, dv)
    s = (torch.einsum("thd,jhd->htj", q_n, k_n) + torch.einsum("thd,jd->htj", q_r, k_r)) * m["scale"]
    i, j = pos[:, None], pos[None, :]
    seen = (i - j >= 0)
    if m.get("mask"):
        seen = seen & (i - j < int(m["mask"]["size"]))
    s = s.masked_fill(~seen[None], float("-inf"))
    sink = W["sink"].to(h.dtype)[:, None, None]
    top = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - top)
    p = e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))       # the sink: no key, no value
    o = torch.einsum("htj,jhd->thd", p, v).reshape(T, H * dv)
    o = store(o * torch.sigmoid(h @ W["g"].T))
    return o @ W["o"].T


def gla(h, W, m, eps, store=_keep):
    """Linear attention with a decay per key channel: S_t = diag(a_t) S_{t-1} + k_t v_t^T,
    o_t = S_t^T q_t, S_{-1} = 0; a = sigmoid(z)^(1/tau)."""
    T = h.shape[0]
    H, dk, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ W["q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ W["k"].T).view(T, H, dk)
    v = (h @ W["v"].T).view(T, H, dv)
    z = (h @ W["a1"].T) @ W["a2"].T + W["a2.b"]
    a = torch.exp(torch.nn.functional.logsigmoid(z) / tau).view(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=h.dtype)
    o = torch.empty(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms_norm(o, W["norm"], eps).reshape(T, H * dv)
    o = store(o * silu(h @ W["g"].T))
    return o @ W["o"].T


MIXERS = {"latent_attention": latent_attention, "gla": gla}


# ---- feed-forwards --------------------------------------------------------------------------------
def dense_ff(h, W, store=_keep):
    return store(gelu_tanh(h @ W["gate"].T) * (h @ W["up"].T)) @ W["down"].T


def routed_ff(h, W, mlp, store=_keep):
    """s = softmax(router h) over all experts; the `top` largest are used, weighted by s itself."""
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    s = torch.softmax(h @ W["router"].T, dim=-1)
    w, idx = torch.topk(s, top, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for r in range(top):
            e = int(idx[t, r])
            out[t] += w[t, r] * (store(gelu_erf(h[t] @ W[f"e{e}.up"].T)) @ W[f"e{e}.down"].T)
    return out


def feed_forward(h, W, mlp, store=_keep):
    if mlp["kind"] == "dense":
        return dense_ff(h, W, store)
    if mlp["kind"] == "moe":
        return routed_ff(h, W, mlp, store)
    raise ValueError(mlp["kind"])


# ---- the model ------------------------------------------------------------------------------------
class PlainKebisun:
    def __init__(self, folder: str = None, config: dict = None, tensors: Dict[str, torch.Tensor] = None):
        if folder is not None:
            with open(f"{folder}/config.json") as f:
                config = json.load(f)
            tensors = read_safetensors(f"{folder}/model.safetensors")
        self.c, self.w = config, tensors

    def _sub(self, prefix, dtype):
        return {k[len(prefix):]: v.to(dtype) for k, v in self.w.items() if k.startswith(prefix)}

    def run(self, ids: Sequence[int], dtype=torch.float64, store=None):
        """(logits [T, vocab], the stream after every layer [L, T, D])."""
        store = store or _keep
        c, eps = self.c, float(self.c["norm"]["eps"])
        x = self.w["embed"][torch.tensor(list(ids), dtype=torch.long)].to(dtype) * float(c["embedding"]["scale"])
        after = []
        for i, layer in enumerate(c["layers"]):
            p = f"l{i}."
            y = MIXERS[layer["type"]](store(x), self._sub(p + "mix.", dtype), layer["mixer"], eps, store)
            x = x + layer_norm(y, self.w[p + "norm1"].to(dtype), eps) * self.w[p + "ls1"].to(dtype)
            if layer.get("mlp"):
                y = feed_forward(store(x), self._sub(p + "mlp.", dtype), layer["mlp"], store)
                x = x + layer_norm(y, self.w[p + "norm2"].to(dtype), eps) * self.w[p + "ls2"].to(dtype)
            after.append(x.clone())
        hn = store(layer_norm(x, self.w["final.norm"].to(dtype), eps))
        return hn @ self.w["head"].to(dtype).T, torch.stack(after)

    def logits(self, ids, dtype=torch.float64, store=None):
        return self.run(ids, dtype, store)[0]
