"""The Kebisun design on the host: configuration reading, the tensor declaration, cache needs, and
the plain implementation against second forms of its own mechanisms (no GPU)."""
import math

import numpy as np
import pytest
import torch

import herbert_rs_b200 as hb
import kebisun_util as K
import plain_kebisun as P
from herbert_rs_b200.cache import SequenceCache
from herbert_rs_b200.errors import ConfigError, WeightError
from herbert_rs_b200.weights.loader import build_model, check_tensors
from herbert_rs_b200.weights.safetensors_io import ModelFiles

LAYERS = [(K.latent(), K.dense()), (K.gla(), K.moe()), (K.latent(window=5), None)]


def test_the_configuration_becomes_a_layer_list():
    cfg = K.config(LAYERS, vocab=99, width=48, emb_scale=2.5, eps=3e-6)
    assert hb.registry.architecture_for(cfg) == "Kebisun"
    spec = hb.config_from_json(cfg).model_spec()
    assert (spec.vocab_size, spec.hidden_size, spec.embedding_scale, len(spec.blocks)) == (99, 48, 2.5, 3)
    a, g, c = (b.mixer for b in spec.blocks)
    assert (a.kind, a.num_heads, a.nope_dim, a.rope_dim, a.v_dim, a.kv_rank, a.q_rank, a.window) == \
        ("latent_attention", 3, 16, 8, 24, 40, 20, 12)
    assert a.scale == cfg["layers"][0]["mixer"]["scale"] and a.norm_eps == 3e-6 and a.sink and a.gate
    assert (a.position.theta, a.position.factor, a.position.original, a.position.fast, a.position.slow) == (10000.0, 4.0, 64, 8.0, 1.0)
    assert (g.kind, g.num_heads, g.key_dim, g.value_dim, g.decay_tau) == ("gla", 2, 24, 40, 8.0) and c.window == 5
    f0, f1, f2 = (b.ffn for b in spec.blocks)
    assert (f0.kind, f0.activation, f0.intermediate_size) == ("swiglu", "gelu_tanh", 72)
    assert (f1.kind, f1.num_experts, f1.top_k, f1.expert_size, f1.renormalize, f1.activation) == ("moe", 5, 2, 24, False, "gelu")
    assert f2 is None and all(b.kind == "sublayer_norm" and b.norm1.kind == "layernorm" for b in spec.blocks)
    assert hb.config_from_json(cfg).to_dict() == cfg


@pytest.mark.parametrize("change,text", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), "rot.dims"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda c: c["layers"][1]["mixer"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][0]["mlp"].update(kind="conv"), "unknown feed-forward"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
])
def test_faults_of_a_configuration_are_named(change, text):
    cfg = K.config(LAYERS)
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        hb.config_from_json(cfg)


def test_tensor_declaration_cache_needs_and_a_wrong_folder(tmp_path):
    cfg = K.config(LAYERS)
    t = K.weights(cfg, decay_rank=5)
    K.write(cfg, t, tmp_path)
    model = build_model(cfg, hb.Runtime("cpu", torch.bfloat16))
    files = ModelFiles(str(tmp_path))
    check_tensors(model, files)                         # the decay's inner size is the tensor's
    files.close()
    assert set(model.param_specs()) == set(t)
    needs = model.cache_needs()
    assert (needs[0].kv.num_kv_heads, needs[0].kv.head_dim, needs[0].kv.window, needs[0].kv.planes) == (1, 48, 12, 1)
    assert needs[1].kv is None and needs[1].state.shape == (2, 24, 40) and needs[1].state.dtype == torch.float32
    cache = SequenceCache(needs, model.reads_cache_of(), num_pages=8, num_slots=2, page_size=16)
    assert len(cache.kv_needs) == 2 and len(cache.state_needs) == 1     # two windows, one state shape
    bad = dict(t)
    bad["l1.mix.a2"] = bad["l1.mix.a2"][:, :4].contiguous()
    del bad["l0.mix.sink"]
    K.write(cfg, bad, tmp_path / "bad")
    files = ModelFiles(str(tmp_path / "bad"))
    with pytest.raises(WeightError, match="l0.mix.sink"):
        check_tensors(model, files)
    files.close()


def test_a_cache_group_of_one_plane_and_a_windowed_release():
    from herbert_rs_b200.cache import CacheNeed, KVNeed
    cache = SequenceCache([CacheNeed(kv=KVNeed(1, 24, 20, planes=1)), CacheNeed(kv=KVNeed(2, 8))], [None, None],
                          num_pages=6, num_slots=2, page_size=16, device="cpu", dtype=torch.float32)
    assert cache.kv[0].shape == (1, 1, 6, 1, 16, 24) and cache.kv[1].shape == (1, 2, 6, 2, 16, 8)
    assert cache.view(0).v is None and cache.view(1).v is not None
    assert cache.bytes_per_token() == 4 * (24 + 2 * 2 * 8)
    s = cache.alloc_slot()
    cache.reserve([(s, 70)])
    cache.advance(s, 70)                                 # the next query, at 70, reads from 51: pages 0..2 are out of reach
    assert [p >= 0 for p in cache.pages_of(s, 0)] == [False, False, False, True, True]
    assert all(p >= 0 for p in cache.pages_of(s, 1))
    cache.check()


# ---- the plain implementation against other forms of the same mechanisms -------------------------------
def _latent_weights(m, D, g):
    H, dn, dr, dv, rk, rq = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64) / math.sqrt(s[-1])  # noqa: E731
    return {"dq": r(rq, D), "dq.norm": 1 + 0.1 * r(rq), "uq": r(H * (dn + dr), rq), "dkv": r(rk + dr, D), "dkv.norm": 1 + 0.1 * r(rk),
            "uk": r(H * dn, rk), "uv": r(H * dv, rk), "sink": torch.randn(H, generator=g, dtype=torch.float64), "g": r(H * dv, D),
            "o": r(D, H * dv)}


def test_plain_latent_attention_against_a_loop_over_single_queries():
    """Token by token, key by key, with explicit keys and values per head."""
    g = torch.Generator().manual_seed(0)
    m = K.latent(window=4, sharp=2.0)["mixer"]
    D, T, eps = 32, 11, 1e-5
    W, h = _latent_weights(m, D, g), torch.randn(T, D, generator=g, dtype=torch.float64)
    ref = P.latent_attention(h, W, m, eps)
    H, dn, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    f, ms = P.rotary_frequencies(m["rot"], torch.float64)

    def turn(u, p):
        out = u.clone()
        for i in range(dr // 2):
            a = p * float(f[i])
            c, s = math.cos(a) * ms, math.sin(a) * ms
            out[i], out[i + dr // 2] = u[i] * c - u[i + dr // 2] * s, u[i + dr // 2] * c + u[i] * s
        return out
    rows = []
    for t in range(T):
        cq = W["dq"] @ h[t]
        cq = cq / torch.sqrt((cq * cq).mean() + eps) * W["dq.norm"]
        q = (W["uq"] @ cq).view(H, dn + dr)
        heads = []
        for hd in range(H):
            num, den = torch.zeros(dv, dtype=torch.float64), math.exp(float(W["sink"][hd]))
            for j in range(max(0, t - 3), t + 1):
                kv = W["dkv"] @ h[j]
                c = kv[:rk] / torch.sqrt((kv[:rk] ** 2).mean() + eps) * W["dkv.norm"]
                k = torch.cat([(W["uk"] @ c).view(H, dn)[hd], turn(kv[rk:], j)])
                qq = torch.cat([q[hd, :dn], turn(q[hd, dn:], t)])
                e = math.exp(float(qq @ k) * m["scale"])
                num += e * (W["uv"] @ c).view(H, dv)[hd]
                den += e
            heads.append(num / den)
        o = torch.cat(heads) * torch.sigmoid(W["g"] @ h[t])
        rows.append(W["o"] @ o)
    assert torch.allclose(torch.stack(rows), ref, atol=1e-10)


def test_plain_gla_against_its_sum_form():
    """o_t = sum over s <= t of (q_t . (prod of decays after s) * k_s) v_s."""
    g = torch.Generator().manual_seed(1)
    m = K.gla(heads=2, dim=6, vdim=5, tau=2.0)["mixer"]
    D, T, R, eps = 16, 9, 3, 1e-5
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64) / math.sqrt(s[-1])  # noqa: E731
    W = {"q": r(12, D), "k": r(12, D), "v": r(10, D), "g": r(10, D), "o": r(D, 10), "norm": 1 + 0.1 * r(5), "a1": r(R, D),
         "a2": r(12, R) * 3, "a2.b": torch.randn(12, generator=g, dtype=torch.float64)}
    h = torch.randn(T, D, generator=g, dtype=torch.float64)
    ref = P.gla(h, W, m, eps)
    q = (h @ W["q"].T).view(T, 2, 6) / math.sqrt(6)
    k, v = (h @ W["k"].T).view(T, 2, 6), (h @ W["v"].T).view(T, 2, 5)
    a = (torch.sigmoid((h @ W["a1"].T) @ W["a2"].T + W["a2.b"]) ** 0.5).view(T, 2, 6)
    o = torch.zeros(T, 2, 5, dtype=torch.float64)
    for t in range(T):
        for s in range(t + 1):
            keep = torch.ones(2, 6, dtype=torch.float64)
            for u in range(s + 1, t + 1):
                keep = keep * a[u]
            o[t] += ((q[t] * keep * k[s]).sum(-1))[:, None] * v[s]
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * W["norm"]
    out = (o.reshape(T, 10) * P.silu(h @ W["g"].T)) @ W["o"].T
    assert torch.allclose(out, ref, atol=1e-10)


def test_plain_small_functions():
    z = torch.linspace(-4, 4, 9, dtype=torch.float64)
    assert torch.allclose(P.gelu_erf(z), torch.nn.functional.gelu(z), atol=1e-12)
    assert torch.allclose(P.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"), atol=1e-12)
    y = torch.randn(3, 10, dtype=torch.float64)
    w = torch.rand(10, dtype=torch.float64)
    assert torch.allclose(P.layer_norm(y, w, 1e-5), torch.nn.functional.layer_norm(y, (10,), w, None, 1e-5), atol=1e-12)
    f, m = P.rotary_frequencies({"base": 100.0, "dims": 8}, torch.float64)
    assert m == 1.0 and np.allclose(f.numpy(), 100.0 ** (-np.arange(4) / 4))
    f2, m2 = P.rotary_frequencies({"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}},
                                  torch.float64)
    # d(4) = 8 ln(16 / (8 pi)) / (2 ln 100) < 0 -> lo 0;  d(1) = 8 ln(16 / (2 pi)) / (2 ln 100) = 0.81 -> hi 1
    assert np.allclose(f2.numpy(), f.numpy() * np.array([1.0, 0.25, 0.25, 0.25])) and abs(m2 - (0.1 * math.log(4.0) + 1)) < 1e-15
