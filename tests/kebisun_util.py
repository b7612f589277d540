"""Small Kebisun configurations and weights for tests.  Nothing here is shared with the library's
compute path: tensors are drawn with torch's generator and written with the container writer.

Weights: matrices N(0, 1/in), norm weights and layer scales 1 + 0.2 N, sinks and decay biases N(0, 1).
Routers are made decisive unless asked otherwise, so that no comparison in bfloat16 rests on a close
call between two experts: the first E channels of the stream carry, for every token id, a ranking of
the experts (in steps of `step`), no sublayer writes to those channels (their layer scales are zero),
and router row e reads channel e with weight 1 beside small random weights elsewhere.
"""
from __future__ import annotations

import copy
import json
import math
import os

import torch

from herbert_rs_b200.weights.safetensors_io import save_file


def latent(heads=3, dim=16, rot=8, vdim=24, kv_rank=40, q_rank=20, window=12, sharp=1.0, scaling=True, base=10000.0,
           original=64, factor=4.0, fast=8.0, slow=1.0):
    rot_cfg = {"base": base, "dims": rot}
    if scaling:
        rot_cfg["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": sharp / math.sqrt(dim + rot), "mask": {"size": window}, "rot": rot_cfg}}


def gla(heads=2, dim=24, vdim=40, tau=8.0):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}}


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=24):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(layers, vocab=131, width=64, emb_scale=3.0, eps=1e-5):
    """layers: list of (mixer entry, mlp entry or None)."""
    return {"architecture": "Kebisun", "vocab": vocab, "width": width, "embedding": {"scale": emb_scale},
            "norm": {"eps": eps}, "layers": [copy.deepcopy(dict(m, mlp=f)) for m, f in layers]}


def _bf16(t):
    return t.to(torch.bfloat16)


def weights(cfg, seed=0, decay_rank=6, decisive_router=True, step=1.5):
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * (gain / math.sqrt(i))

    def vec(n, mean=1.0, std=0.2):
        return mean + std * torch.randn(n, generator=g)

    w = {"embed": mat(V, D, gain=math.sqrt(D) * 0.5), "head": mat(V, D), "final.norm": vec(D)}
    E = max((l["mlp"]["router"]["experts"] for l in cfg["layers"] if l.get("mlp") and l["mlp"]["kind"] == "moe"), default=0)
    if E and decisive_router:
        assert E < D
        for tok in range(V):
            ranks = torch.randperm(E, generator=g).double()
            w["embed"][tok, :E] = ranks * step / cfg["embedding"]["scale"]
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        w[p + "norm1"], w[p + "ls1"] = vec(D), vec(D)
        if l["type"] == "latent_attention":
            H, dn, dr, dv, rk, rq = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            w.update({p + "mix.dq": mat(rq, D), p + "mix.dq.norm": vec(rq), p + "mix.uq": mat(H * (dn + dr), rq, 2.0),
                      p + "mix.dkv": mat(rk + dr, D, 2.0), p + "mix.dkv.norm": vec(rk), p + "mix.uk": mat(H * dn, rk, 2.0),
                      p + "mix.uv": mat(H * dv, rk), p + "mix.sink": vec(H, 0.0, 1.0), p + "mix.g": mat(H * dv, D),
                      p + "mix.o": mat(D, H * dv)})
        else:
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            w.update({p + "mix.q": mat(H * dk, D), p + "mix.k": mat(H * dk, D), p + "mix.v": mat(H * dv, D),
                      p + "mix.g": mat(H * dv, D), p + "mix.o": mat(D, H * dv), p + "mix.norm": vec(dv),
                      p + "mix.a1": mat(decay_rank, D), p + "mix.a2": mat(H * dk, decay_rank, 2.0),
                      p + "mix.a2.b": vec(H * dk, 1.0, 1.5)})
        f = l.get("mlp")
        if f:
            w[p + "norm2"], w[p + "ls2"] = vec(D), vec(D)
            if f["kind"] == "dense":
                w.update({p + "mlp.gate": mat(f["ff"], D, 2.0), p + "mlp.up": mat(f["ff"], D), p + "mlp.down": mat(D, f["ff"])})
            else:
                n = f["router"]["experts"]
                for e in range(n):
                    w[p + f"mlp.e{e}.up"] = mat(f["expert"]["ff"], D, 2.0)
                    w[p + f"mlp.e{e}.down"] = mat(D, f["expert"]["ff"])
                r = mat(n, D, 2.0)
                if decisive_router:
                    r = r * 0.15
                    r[:, :E] = 0.0
                    r[:, :n] = torch.eye(n)
                w[p + "mlp.router"] = r
        if E and decisive_router:
            for k in ("ls1", "ls2"):
                if p + k in w:
                    w[p + k][:E] = 0.0
    return {k: _bf16(v) for k, v in w.items()}


def write(cfg, tensors, folder):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file(dict(tensors), os.path.join(folder, "model.safetensors"))
    return str(folder)


def make(folder, layers, seed=0, **kw):
    """Write a model folder; returns (folder, plain model)."""
    import plain_kebisun as P
    wkw = {k: kw.pop(k) for k in ("decay_rank", "decisive_router", "step") if k in kw}
    cfg = config(layers, **kw)
    t = weights(cfg, seed, **wkw)
    write(cfg, t, folder)
    return str(folder), P.PlainKebisun(str(folder))
