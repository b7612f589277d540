"""Small Votapel configurations and weights for tests.  Nothing here is shared with the library's
compute path: tensors are drawn with torch's generator and written with the container writer.

Weights: matrices N(0, 1/in), norm weights 0.2 N around zero, biases 0.3 N, sinks N(0, 1), position
vectors 0.3 N.

Routers are made decisive unless asked otherwise, so that no comparison in bfloat16 rests on a close
call between two experts or two groups: the first E channels of the stream carry, for every token
id, one router logit per expert; nothing writes to those channels (the position table, the output
products' rows and the norm weights are zero there), and router row e reads channel e with weight 1
beside tiny random weights elsewhere.  The logits of a token id are drawn again until the choice of
groups and of experts holds with a margin for every factor the norm may put on them.
"""
from __future__ import annotations

import copy
import json
import math
import os

import torch

from herbert_rs_b200.weights.safetensors_io import save_file

NORM_FACTORS = (0.25, 0.4, 0.6, 0.8, 1.0, 1.3)       # what 1 / rms(x) can be in these models


def attention(heads=4, kv_heads=2, dim=16, scale=None, softcap=8.0, coef=0.4, every=5, sharp=1.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
         "scale": sharp / math.sqrt(dim) if scale is None else scale}
    if softcap is not None:
        m["softcap"] = softcap
    if coef is not None:
        m["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention", "mixer": m}


def moe(experts=6, top=2, ff=24, groups=3, keep=2, scale=1.5, shared=40):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if groups is not None:
        f["router"]["groups"] = {"count": groups, "keep": keep}
    if shared is not None:
        f["shared"] = {"ff": shared}
    return f


def config(layers, vocab=131, width=64, eps=1e-5, mult=0.6, max_positions=512):
    """layers: list of (mixer entry, mlp entry or None)."""
    return {"architecture": "Votapel", "vocab": vocab, "width": width, "max_positions": max_positions,
            "norm": {"eps": eps}, "residual_mult": mult, "layers": [copy.deepcopy(dict(m, mlp=f)) for m, f in layers]}


def route_with_margins(z, groups, keep, top):
    """(chosen experts, smallest margin) for router logits z [E] (float64): the margin is the smaller of the
    gap between the last kept and the first dropped group's score and the gap between the last chosen and
    the first not chosen expert's score among the kept groups' experts."""
    s = torch.sigmoid(z)
    E = s.shape[0]
    size = E // groups
    gs = torch.stack([torch.sort(s[g * size:(g + 1) * size], descending=True).values[:2].sum() for g in range(groups)])
    order = torch.argsort(gs, descending=True, stable=True)
    margin = float(gs[order[keep - 1]] - gs[order[keep]]) if keep < groups else 1.0
    open_ = [e for e in range(E) if e // size in order[:keep].tolist()]
    ranked = sorted(open_, key=lambda e: (-float(s[e]), e))
    if top < len(ranked):
        margin = min(margin, float(s[ranked[top - 1]] - s[ranked[top]]))
    return ranked[:top], margin


def decisive_logits(g, experts, groups, keep, top, need=0.04):
    """Every other draw gives one group a single high logit beside very low ones (its score stays near 1
    while the expert itself is among the best), so that the groups change the choice for many tokens."""
    size = experts // groups
    while True:
        z = (torch.rand(experts, generator=g, dtype=torch.float64) * 2 - 1) * 3.0
        if size > 1 and groups > 1 and float(torch.rand(1, generator=g)) < 0.5:
            at = int(torch.randint(groups, (1,), generator=g)) * size
            z[at:at + size] = -2.6 - 0.4 * torch.rand(size, generator=g, dtype=torch.float64)
            z[at + int(torch.randint(size, (1,), generator=g))] = 2.6 + 0.4 * float(torch.rand(1, generator=g))
        if all(route_with_margins(z * f, groups, keep, top)[1] >= need for f in NORM_FACTORS):
            return z


def _bf16(t):
    return t.to(torch.bfloat16)


def weights(cfg, seed=0, decisive_router=True):
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * (gain / math.sqrt(i))

    def vec(n, mean=0.0, std=0.2):
        return mean + std * torch.randn(n, generator=g)

    w = {"embed": mat(V, D, gain=math.sqrt(D)), "pos": torch.randn(cfg["max_positions"], D, generator=g) * 0.3,
         "head": mat(V, D), "final.norm": vec(D)}
    routed = [l["mlp"]["router"] for l in cfg["layers"] if l.get("mlp")]
    E = max((r["experts"] for r in routed), default=0)
    if E and decisive_router:
        assert E < D and all(r == routed[0] for r in routed), "decisive routers share one shape"
        r0 = routed[0]
        gr = r0.get("groups") or {"count": 1, "keep": 1}
        for tok in range(V):
            w["embed"][tok, :E] = decisive_logits(g, E, gr["count"], gr["keep"], r0["top"]).float()
        w["pos"][:, :E] = 0.0
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        H, G, d = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
        w[p + "norm1"] = vec(D)
        w.update({p + "mix.q": mat(H * d, D), p + "mix.q.b": vec(H * d, 0.0, 0.3), p + "mix.k": mat(G * d, D, 1.5),
                  p + "mix.k.b": vec(G * d, 0.0, 0.3), p + "mix.sink": vec(H, 0.0, 1.0), p + "mix.o": mat(D, H * d)})
        f = l.get("mlp")
        outs = [p + "mix.o"]
        if f:
            n, ff = f["router"]["experts"], f["expert"]["ff"]
            for e in range(n):
                w[p + f"mlp.e{e}.gate"], w[p + f"mlp.e{e}.up"] = mat(ff, D, 2.0), mat(ff, D)
                w[p + f"mlp.e{e}.down"] = mat(D, ff)
                outs.append(p + f"mlp.e{e}.down")
            r = mat(n, D, 2.0)
            if decisive_router:
                r = r * 0.01
                r[:, :E] = 0.0
                r[:, :n] = torch.eye(n)
            w[p + "mlp.router"] = r
            if f.get("shared"):
                sf = f["shared"]["ff"]
                w.update({p + "mlp.shared.gate": mat(sf, D, 2.0), p + "mlp.shared.up": mat(sf, D), p + "mlp.shared.down": mat(D, sf)})
                outs.append(p + "mlp.shared.down")
        if E and decisive_router:
            w[p + "norm1"][:E] = 0.0
            for name in outs:
                w[name][:E] = 0.0
    return {k: _bf16(v) for k, v in w.items()}


def write(cfg, tensors, folder):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file(dict(tensors), os.path.join(folder, "model.safetensors"))
    return str(folder)


def make(folder, layers, seed=0, decisive_router=True, **kw):
    """Write a model folder; returns (folder, plain model)."""
    import plain_votapel as P
    cfg = config(layers, **kw)
    write(cfg, weights(cfg, seed, decisive_router), folder)
    return str(folder), P.PlainVotapel(str(folder))
