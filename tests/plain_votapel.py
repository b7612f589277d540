"""A plain, slow implementation of the Votapel decoder: whole sequences, no cache, no batching, one
function per mechanism, written from the design's equations.  It shares no code with the library:
config.json and the safetensors file are parsed here (the container reader is the other plain
model's) and everything is computed with torch on the CPU.

The design in this file's notation (T tokens, D = width, positions p = 0, 1, ... in a sequence):

  x_0[p] = E[token_p] + P[p]                                 (a learned vector per position)
  a layer:  h = N(x);  x <- x + m * (mixer(h) + ff(h))       (one norm, both sublayers read it; a
            layer may lack ff;  N(x) = x / sqrt(mean(x^2) + eps) * (1 + w): weights lie around 0)
  logits = head N_final(x)

  mixer "attention": H query heads, G key/value heads (query head i reads head i // (H/G)), head size d
      q = Wq h + bq, k = Wk h + bk, and the values ARE the keys (v = k; no value product)
      q_p <- q_p * (1 + c * ln(floor((p + 1) / n) + 1))        (a temperature that grows with p)
      s = (q . k) * scale;  s <- cap * tanh(s / cap);  causal
      weights a_j = exp(s_j) / (exp(sink_i) + sum_j' exp(s_j'))  (a learned number per head sits in
      the denominator only);  out = Wo concat_i(sum_j a_j v_j)
  ff "moe": z = R h, s = sigmoid(z).  The E experts form n_g groups of neighbours; a group's score is
      the sum of its two largest s; only experts of the `keep` best groups can be chosen; of those the
      `top` largest s are chosen (ties to the lower index); weight = s * router scale, no
      renormalisation;  expert(h) = Wd (silu(Wg h) * (Wu h));  a shared expert of the same form
      runs for every token and is added.

`dtype` is the dtype of all arithmetic (float64 for a ground truth).  Weights are used as stored
(bfloat16 values widened exactly).  `store`, where given, is applied to every activation that an
engine would keep in its activation dtype between two kernels (`bf16_storage` rounds those to
bfloat16): what the number format alone does to the logits follows from it.
"""

from __future__ import annotations

import json
import math
import os
from typing import Sequence

import torch

from plain_kebisun import bf16_storage, read_safetensors  # noqa: F401  (container reader and rounding only)


def _keep(t):
    return t


# ---- one function per mechanism ---------------------------------------------------------------
def offset_rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * (1 + w)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1) per position."""
    p = torch.as_tensor(positions, dtype=torch.int64)
    return 1.0 + coef * torch.log(torch.div(p + 1, every, rounding_mode="floor").double() + 1.0)


def capped(s, cap):
    return s if cap is None else cap * torch.tanh(s / cap)


def sink_softmax_row(scores, sink):
    """Weights of one query's scores (a vector) with exp(sink) added to the denominator."""
    m = max(float(scores.max()), float(sink)) if sink is not None else float(scores.max())
    e = torch.exp(scores - m)
    den = e.sum() + (math.exp(float(sink) - m) if sink is not None else 0.0)
    return e / den


def attention_heads(q, k, v, scale, cap, sink, positions=None):
    """q [T, H, d], k, v [T, G, d] of one sequence from its first token on -> [T, H, d]; key by key,
    query by query.  `positions` only matters through causality: token t sees tokens 0..t."""
    T, H, d = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for i in range(H):
        g = i // (H // G)
        for t in range(T):
            s = (k[: t + 1, g] @ q[t, i]) * scale
            a = sink_softmax_row(capped(s, cap), None if sink is None else sink[i])
            out[t, i] = a @ v[: t + 1, g]
    return out


def attention_mixer(h, w, m, positions, dtype, store=_keep):
    """The whole mixer on normed input h [T, D]; w: the layer's tensors by local name."""
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = h @ w["q"].to(dtype).T + w["q.b"].to(dtype)
    k = h @ w["k"].to(dtype).T + w["k.b"].to(dtype)
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(positions, qt["coef"], qt["every"]).to(dtype)[:, None]
    q, k = store(q).view(T, H, d), store(k).view(T, G, d)
    sink = w["sink"].to(dtype) if "sink" in w else None
    o = attention_heads(q, k, k, m["scale"], m.get("softcap"), sink)
    return store(o.reshape(T, -1)) @ w["o"].to(dtype).T


def gated_expert(h, gate, up, down, store=_keep):
    return store(silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(scores, groups, keep, top):
    """scores [E] of one token -> the chosen experts, best first.  Groups of neighbours; a group's
    score is the sum of its two largest scores (of its one, if it has one)."""
    E = scores.shape[0]
    size = E // groups
    gs = []
    for g in range(groups):
        part = sorted((float(x) for x in scores[g * size:(g + 1) * size]), reverse=True)
        gs.append(sum(part[:2]))
    kept = sorted(range(groups), key=lambda g: (-gs[g], g))[:keep]
    allowed = [e for e in range(E) if e // size in kept]
    return sorted(allowed, key=lambda e: (-float(scores[e]), e))[:top]


def routed_ff(h, w, f, dtype, store=_keep, log=None):
    """The mixture on normed input h [T, D]; w: the feed-forward's tensors by local name.  `log`, a list,
    receives (router logits [E], chosen experts) per token."""
    r = f["router"]
    E, top = r["experts"], r["top"]
    gr = r.get("groups") or {"count": 1, "keep": 1}
    z = h.to(torch.float64) @ w["router"].to(torch.float64).T
    s = torch.sigmoid(z)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=dtype)
    for t in range(h.shape[0]):
        chosen = route(s[t], gr["count"], gr["keep"], top)
        if log is not None:
            log.append((z[t].clone(), chosen))
        for e in chosen:
            y = gated_expert(h[t:t + 1], w[f"e{e}.gate"].to(dtype), w[f"e{e}.up"].to(dtype), w[f"e{e}.down"].to(dtype), store)
            out[t] += (s[t, e] * r.get("scale", 1.0)).to(dtype) * y[0]
    if f.get("shared"):
        out = out + gated_expert(h, w["shared.gate"].to(dtype), w["shared.up"].to(dtype), w["shared.down"].to(dtype), store)
    return out


# ---- the model ----------------------------------------------------------------------------------
class PlainVotapel:
    def __init__(self, folder: str = None, config: dict = None, tensors: dict = None):
        if folder is not None:
            with open(os.path.join(folder, "config.json")) as f:
                config = json.load(f)
            tensors = read_safetensors(os.path.join(folder, "model.safetensors"))
        self.cfg, self.w = config, tensors
        self.vocab = self.cfg["vocab"]

    def _sub(self, prefix):
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def hidden(self, ids: Sequence[int], dtype=torch.float64, store=_keep, layers_out=None, routes_out=None):
        """The residual stream after the last layer, [T, D]; `layers_out`, a list, receives it after
        every layer, `routes_out` every token's router logits and choice, layer by layer."""
        c = self.cfg
        T = len(ids)
        pos = list(range(T))
        x = self.w["embed"].to(dtype)[torch.tensor(ids)] + self.w["pos"].to(dtype)[:T]
        eps, mult = c["norm"]["eps"], c.get("residual_mult", 1.0)
        for i, layer in enumerate(c["layers"]):
            h = store(offset_rms_norm(x, self.w[f"l{i}.norm1"].to(dtype), eps))
            y = attention_mixer(h, self._sub(f"l{i}.mix."), layer["mixer"], pos, dtype, store)
            if layer.get("mlp"):
                y = y + routed_ff(h, self._sub(f"l{i}.mlp."), layer["mlp"], dtype, store, routes_out)
            x = x + mult * y
            if layers_out is not None:
                layers_out.append(x.clone())
        return x

    def logits(self, ids: Sequence[int], dtype=torch.float64, store=_keep) -> torch.Tensor:
        """[T, vocab] float32."""
        x = self.hidden(ids, dtype, store)
        hn = store(offset_rms_norm(x, self.w["final.norm"].to(dtype), self.cfg["norm"]["eps"]))
        return (hn @ self.w["head"].to(dtype).T).to(torch.float32)


def greedy(model: PlainVotapel, prompt: Sequence[int], n: int, dtype=torch.float64) -> list:
    ids, out = list(prompt), []
    for _ in range(n):
        tok = int(model.logits(ids, dtype)[-1].argmax())
        out.append(tok)
        ids.append(tok)
    return out
