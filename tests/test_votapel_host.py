"""The Votapel design without a GPU: configuration reading and its error messages, the tensor
declaration, cache needs, and the plain implementation against second forms of its own mechanisms."""
import copy
import math

import numpy as np
import pytest
import torch

import herbert_rs_b200 as hb
import plain_votapel as P
import votapel_util as U
from herbert_rs_b200.config.votapel import VotapelConfig
from herbert_rs_b200.errors import ConfigError
from herbert_rs_b200.weights.loader import build_model


def test_configuration_is_read_from_the_nested_keys():
    cfg = U.config([(U.attention(heads=6, kv_heads=3, dim=24, softcap=11.0, coef=0.25, every=7), U.moe(experts=8, top=3, groups=4, keep=2)),
                    (U.attention(heads=2, kv_heads=2, dim=40, softcap=None, coef=None), None)], vocab=99, width=72, mult=0.35,
                   max_positions=300)
    spec = VotapelConfig.from_dict(cfg).model_spec()
    assert (spec.vocab_size, spec.hidden_size, spec.max_position, spec.position_table_name) == (99, 72, 300, "pos")
    b0, b1 = spec.blocks
    assert b0.kind == "parallel" and b0.residual_mult == 0.35 and b0.norm1.weight_offset == 1.0 and b0.norm1.eps == 1e-5
    m = b0.mixer
    assert (m.num_heads, m.num_kv_heads, m.head_dim, m.softcap, m.q_temperature) == (6, 3, 24, 11.0, (0.25, 7))
    assert m.values_are_keys and m.bias and m.sink and m.position is None and m.window is None
    f = b0.ffn
    assert (f.num_experts, f.top_k, f.groups, f.keep_groups, f.group_top, f.weight_scale) == (8, 3, 4, 2, 2, 1.5)
    assert f.gated and f.score == "sigmoid" and not f.renormalize and f.shared.intermediate_size == 40
    assert b1.ffn is None and b1.mixer.softcap is None and b1.mixer.q_temperature is None
    assert hb.registry.architecture_for(cfg) == "Votapel"


@pytest.mark.parametrize("edit,message", [
    (lambda c: c.update(max_positions=0), "max_positions"),
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(experts=7), "multiple of groups.count"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=4), "exceeds groups.count"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "exceeds the 4 experts"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "unknown feed-forward kind"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
])
def test_configuration_errors_name_the_key(edit, message):
    cfg = U.config([(U.attention(), U.moe())])
    edit(cfg)
    with pytest.raises(ConfigError, match=message):
        VotapelConfig.from_dict(cfg)


def test_declared_tensors_and_cache_need(tmp_path):
    cfg = U.config([(U.attention(heads=4, kv_heads=2, dim=16), U.moe(experts=4, top=1, groups=2, keep=1, shared=None)),
                    (U.attention(heads=3, kv_heads=1, dim=8), None)])
    model = build_model(cfg, hb.Runtime("cpu", torch.bfloat16))
    specs = model.param_specs()
    assert set(specs) == set(U.weights(cfg))
    for name, t in U.weights(cfg).items():
        assert tuple(specs[name].shape) == tuple(t.shape), name
    assert specs["pos"].shape == (512, 64) and specs["l0.mix.q.b"].role == "vector" and "l0.mlp.shared.gate" not in specs
    needs = model.cache_needs()
    assert needs[0].kv.planes == 1 and (needs[0].kv.num_kv_heads, needs[0].kv.head_dim) == (2, 16)
    assert (needs[1].kv.num_kv_heads, needs[1].kv.head_dim, needs[1].kv.window) == (1, 8, None)
    assert model.graph_safe
    U.write(cfg, U.weights(cfg), tmp_path)
    assert P.PlainVotapel(str(tmp_path)).logits([1, 2, 3]).shape == (3, 131)


def test_a_position_table_whose_length_only_the_tensor_gives(tmp_path):
    cfg = U.config([(U.attention(), None)], max_positions=77)
    t = U.weights(cfg)
    del cfg["max_positions"]
    model = build_model(cfg, hb.Runtime("cpu", torch.bfloat16))
    assert model.param_specs()["pos"].shape == (-1, 64)
    from herbert_rs_b200.weights.loader import fill_model
    fill_model(model, lambda name: t[name], model.rt)
    assert model.longest_sequence() == 77


def test_a_missing_or_misshapen_tensor_is_reported(tmp_path):
    from herbert_rs_b200.errors import WeightError
    from herbert_rs_b200.weights.loader import check_tensors
    from herbert_rs_b200.weights.safetensors_io import ModelFiles
    cfg = U.config([(U.attention(), U.moe())])
    t = U.weights(cfg)
    del t["l0.mix.sink"]
    t["l0.mix.k.b"] = t["l0.mix.k.b"][:-1].contiguous()
    U.write(cfg, t, tmp_path)
    files = ModelFiles(str(tmp_path))
    with pytest.raises(WeightError) as e:
        check_tensors(build_model(cfg, hb.Runtime("cpu", torch.bfloat16)), files)
    files.close()
    assert "l0.mix.sink" in str(e.value) and "l0.mix.k.b" in str(e.value)


# ---- the plain implementation against second forms of its mechanisms --------------------------------
def test_attention_against_a_matrix_form():
    g = torch.Generator().manual_seed(0)
    T, H, G, d = 23, 4, 2, 8
    q, k = torch.randn(T, H, d, generator=g, dtype=torch.float64) * 2, torch.randn(T, G, d, generator=g, dtype=torch.float64)
    sink = torch.randn(H, generator=g, dtype=torch.float64)
    got = P.attention_heads(q, k, k, 0.4, 3.0, sink)
    kk = k.repeat_interleave(H // G, dim=1)
    s = 3.0 * torch.tanh(torch.einsum("thd,jhd->htj", q, kk) * 0.4 / 3.0)
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), -math.inf)
    full = torch.cat([s, sink[:, None, None].expand(H, T, 1)], dim=-1)           # the sink as one more column ...
    a = torch.softmax(full, -1)[..., :T]                                         # ... that has no value
    ref = torch.einsum("htj,jhd->thd", a, kk)
    assert (got - ref).abs().max() < 1e-12
    assert float(a.sum(-1).max()) < 1.0                                          # the weights do not sum to one


def test_query_temperature_steps_at_multiples_of_its_period():
    f = P.query_temperature([0, 3, 4, 8, 9, 13, 14, 49], 0.5, 5)
    want = [1.0, 1.0, 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(3), 1 + 0.5 * math.log(3),
            1 + 0.5 * math.log(4), 1 + 0.5 * math.log(11)]
    assert np.allclose(f.numpy(), want, rtol=0, atol=1e-15)


def test_routing_by_groups_differs_from_plain_top_k_and_never_leaves_the_kept_groups():
    g = torch.Generator().manual_seed(1)
    differs = 0
    for _ in range(300):
        s = torch.rand(12, generator=g, dtype=torch.float64)
        chosen = P.route(s, 4, 2, 3)
        sums = [float(torch.sort(s[i * 3:(i + 1) * 3], descending=True).values[:2].sum()) for i in range(4)]
        kept = sorted(range(4), key=lambda i: -sums[i])[:2]
        assert all(e // 3 in kept for e in chosen) and len(set(chosen)) == 3
        assert chosen == U.route_with_margins(torch.logit(s), 4, 2, 3)[0]
        differs += sorted(chosen) != sorted(torch.topk(s, 3).indices.tolist())
    assert differs > 30
    assert P.route(torch.tensor([0.9, 0.1, 0.6, 0.6, 0.5, 0.5]), 3, 1, 2) == [2, 3]      # 1.0 < 1.2: the best single expert loses
    assert P.route(torch.tensor([0.3, 0.7, 0.2]), 3, 2, 1) == [1]                         # groups of one: the score itself
    assert P.route(torch.tensor([0.5, 0.5, 0.5, 0.5]), 2, 1, 2) == [0, 1]                 # ties go to the lower index


def test_decisive_routers_hold_their_margin_in_the_written_models(tmp_path):
    d, pm = U.make(tmp_path, [(U.attention(), U.moe()), (U.attention(heads=2, kv_heads=1), U.moe())], seed=5)
    ids = np.random.default_rng(0).integers(0, 131, 80).tolist()
    routes = []
    pm.hidden(ids, routes_out=routes)
    assert len(routes) == 2 * 80
    differs = 0
    for z, chosen in routes:
        again, margin = U.route_with_margins(z, 3, 2, 2)
        assert again == chosen and margin > 0.02
        differs += sorted(chosen) != sorted(torch.topk(z, 2).indices.tolist())
    assert differs > 5         # the groups change the choice for some tokens


def test_the_offset_norm_and_the_parallel_sum():
    g = torch.Generator().manual_seed(2)
    x, w = torch.randn(5, 16, generator=g, dtype=torch.float64), torch.randn(16, generator=g, dtype=torch.float64) * 0.1
    ref = torch.nn.functional.rms_norm(x, (16,), 1.0 + w, 1e-5)
    assert (P.offset_rms_norm(x, w, 1e-5) - ref).abs().max() < 1e-12
    assert (P.silu(x) - torch.nn.functional.silu(x)).abs().max() < 1e-12


def test_leaving_out_one_mechanism_changes_the_logits(tmp_path):
    """The small models are sensitive to every mechanism: without the sink, the cap, the temperature, the
    position vectors, the groups or the residual factor the plain logits move by far more than any bound."""
    d, pm = U.make(tmp_path, [(U.attention(sharp=2.0), U.moe()), (U.attention(), U.moe())], seed=3)
    ids = np.random.default_rng(1).integers(0, 131, 40).tolist()
    ref = pm.logits(ids)

    def variant(edit_cfg=None, edit_w=None):
        cfg, w = copy.deepcopy(pm.cfg), dict(pm.w)
        if edit_cfg:
            edit_cfg(cfg)
        if edit_w:
            edit_w(w)
        return float((P.PlainVotapel(config=cfg, tensors=w).logits(ids) - ref).abs().max())

    assert variant(edit_w=lambda w: w.update({"l0.mix.sink": w["l0.mix.sink"] - 30.0})) > 0.05
    assert variant(lambda c: c["layers"][0]["mixer"].pop("softcap")) > 0.05
    assert variant(lambda c: c["layers"][0]["mixer"].pop("q_temp")) > 0.05
    assert variant(lambda c: c["layers"][0]["mixer"]["q_temp"].update(every=6)) > 0.01
    assert variant(edit_w=lambda w: w.update({"pos": torch.zeros_like(w["pos"])})) > 0.05
    assert variant(lambda c: c["layers"][0]["mlp"]["router"].pop("groups")) > 0.05
    assert variant(lambda c: c.update(residual_mult=1.0)) > 0.05
    assert variant(lambda c: c["layers"][1]["mlp"].pop("shared")) > 0.05
