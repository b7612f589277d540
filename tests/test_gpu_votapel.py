"""The Votapel design in the engine against the plain implementation (`plain_votapel.py`): every
mechanism alone, prompts against decoding, prompts in pieces, unequal batches, slots and pages that
are used again, far keys and page borders, the first tokens, long decoding, other sizes, greedy
generation through the library's entry points."""
import math

import numpy as np
import pytest
import torch

import herbert_rs_b200 as hb
import plain_votapel as P
import votapel_util as U
from gpu_util import (DTYPES, assert_close, bound_for, engine_for, replay_batches, replay_tail_one_by_one, replay_whole,
                      sensitivity_bound, to_np)
from herbert_rs_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def ids_for(rng, vocab, n):
    return rng.integers(0, vocab, n).tolist()


def td_of(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


@pytest.fixture(scope="module")
def mixed(tmp_path_factory):
    """Layers of different head counts and sizes (each bfloat16 attention kernel is met), one without a
    feed-forward, one without cap and temperature."""
    layers = [(U.attention(heads=4, kv_heads=2, dim=16), U.moe()),
              (U.attention(heads=2, kv_heads=1, dim=64, every=3, coef=0.7), None),
              (U.attention(heads=3, kv_heads=3, dim=24, softcap=None, coef=None), U.moe()),
              (U.attention(heads=2, kv_heads=2, dim=128, softcap=3.0, every=50), U.moe())]
    return U.make(tmp_path_factory.mktemp("votapel_mixed"), layers, seed=3)


# ---- each mechanism alone -------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim", [48, 200, 1100, 4500])
def test_scaled_residual_sum_and_the_next_norm(dtype, dim):
    g = torch.Generator().manual_seed(dim)
    y, x = (torch.randn(6, dim + 8, generator=g) * 2).to(DEV), torch.randn(6, dim, generator=g).to(DEV)
    w = (0.2 * torch.randn(dim, generator=g)).to(DEV)
    x1, h = x.clone(), torch.empty(6, dim, dtype=td_of(dtype), device=DEV)
    ops.scaled_residual_norm(y[:, :dim], 0.7, x1, 1.0 + w, h, 1e-5)
    ref = x.double().cpu() + 0.7 * y[:, :dim].double().cpu()
    assert_close(to_np(x1), ref.numpy(), "float32", "sum")
    assert_close(to_np(h), P.offset_rms_norm(ref, w.double().cpu(), 1e-5).numpy(), dtype, "next norm")
    x2 = x.clone()
    ops.scaled_residual_norm(y[:, :dim], -1.25, x2)
    assert_close(to_np(x2), (x.double().cpu() - 1.25 * y[:, :dim].double().cpu()).numpy(), "float32", "sum alone")


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_with_position_vectors(dtype):
    g = torch.Generator().manual_seed(1)
    td = td_of(dtype)
    table, pos = torch.randn(50, 40, generator=g).to(td).to(DEV), torch.randn(30, 40, generator=g).to(td).to(DEV)
    ids = torch.tensor([3, 49, 0, 3, 17], dtype=torch.int32, device=DEV)
    at = torch.tensor([0, 29, 5, 6, 1], dtype=torch.int32, device=DEV)
    out = torch.zeros(5, 40, device=DEV)
    ops.embed(table, ids, out, 1.0, pos, at)
    ref = table.double()[ids.long()] + pos.double()[at.long()]
    assert np.abs(to_np(out) - ref.cpu().numpy()).max() < 1e-6
    ops.embed(table, ids, out, 2.0)
    assert np.abs(to_np(out) - 2.0 * table.double()[ids.long()].cpu().numpy()).max() < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("with_v", [False, True])
def test_bias_temperature_and_cache_write(dtype, with_v):
    """Positions just below, at and above multiples of the temperature's period; tokens of two sequences in
    pages that are not in order; a row with and without a value part."""
    td = td_of(dtype)
    g = torch.Generator().manual_seed(2)
    H, G, d, page = 3, 2, 12, 16
    every, coef = 7, 0.6
    pos = [0, 5, 6, 7, 12, 13, 14, 15, 16, 17, 48, 49, 31, 32]
    seq = [0] * 12 + [1] * 2
    T, width = len(pos), (H + G * (2 if with_v else 1)) * d
    rows, bias = torch.randn(T, width, generator=g), torch.randn(width, generator=g) * 0.5
    pages = torch.tensor([[5, 2, 7, 0], [3, 1, 6, 4]], dtype=torch.int32)
    cache = torch.zeros(2, 8, G, page, d, dtype=td, device=DEV)
    q = torch.zeros(T, H * d, dtype=td, device=DEV)
    ops.qk_prepare_cache(rows.to(DEV), bias.to(DEV), q, coef, every, torch.tensor(seq, dtype=torch.int32, device=DEV),
                         torch.tensor(pos, dtype=torch.int32, device=DEV), pages.to(DEV), cache[0], cache[1] if with_v else None,
                         H, G, d, page)
    full = rows.double() + bias.double()
    f = P.query_temperature(pos, coef, every)
    assert f[2] > f[1] == 1.0 and f[5] > f[4] and f[9] == f[8] == f[7] == f[6]          # steps at 6, 13, 20, ...
    assert_close(to_np(q), (full[:, :H * d] * f[:, None]).numpy(), dtype, "q")
    for t in range(T):
        p = int(pages[seq[t], pos[t] // page])
        for plane in range(2 if with_v else 1):
            want = full[t, (H + plane * G) * d:(H + (plane + 1) * G) * d].view(G, d)
            assert_close(to_np(cache[plane, p, :, pos[t] % page]), want.numpy(), dtype, f"cache plane {plane} token {t}")
    assert int((cache != 0).sum()) == T * G * d * (2 if with_v else 1)                    # and nothing else was written
    q2 = torch.zeros_like(q)
    ops.qk_prepare_cache(rows.to(DEV), None, q2, 0.0, 0, torch.tensor(seq, dtype=torch.int32, device=DEV),
                         torch.tensor(pos, dtype=torch.int32, device=DEV), pages.to(DEV), cache[0], None, H, G, d, page,
                         write_cache=False)
    assert_close(to_np(q2), rows[:, :H * d].double().numpy(), dtype, "q without bias and temperature")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top,groups,keep", [(12, 3, 4, 2), (6, 2, 3, 2), (8, 4, 1, 1), (4, 1, 4, 1), (5, 5, 5, 5), (64, 6, 8, 3)])
def test_router_with_groups_and_gated_experts(dtype, experts, top, groups, keep):
    td = td_of(dtype)
    g = torch.Generator().manual_seed(experts + top)
    T, D, F = 45, 48, 24
    h = torch.randn(T, D, generator=g).to(td)
    r = (torch.randn(experts, D, generator=g) * 0.4).to(torch.bfloat16).to(td)
    gate = (torch.randn(experts, F, D, generator=g) * 2 / math.sqrt(D)).to(torch.bfloat16).to(td)
    up = (torch.randn(experts, F, D, generator=g) / math.sqrt(D)).to(torch.bfloat16).to(td)
    down = (torch.randn(experts, D, F, generator=g) / math.sqrt(F)).to(torch.bfloat16).to(td)
    z = h.double() @ r.double().T
    sure = [t for t in range(T) if U.route_with_margins(z[t], groups, keep, top)[1] > 1e-3]
    assert len(sure) > T // 2
    ids = torch.zeros(T, top, dtype=torch.int32, device=DEV)
    wts = torch.zeros(T, top, device=DEV)
    ops.moe_route(h.to(DEV), r.to(DEV), ids, wts, top, False, 1, groups, keep, 2, 1.75)
    s = torch.sigmoid(z)
    for t in sure:
        want = P.route(s[t], groups, keep, top)
        assert ids[t].tolist() == want, (t, ids[t].tolist(), want)
        assert np.abs(to_np(wts[t]) - 1.75 * s[t, want].numpy()).max() < 1e-5
    # the experts with the router's own choice (whatever it was), in both kernels
    W = {"router": r.double()}
    for e in range(experts):
        W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"] = gate[e].double(), up[e].double(), down[e].double()
    ref = torch.zeros(T, D, dtype=torch.float64)
    for t in range(T):
        for j in range(top):
            e = int(ids[t, j])
            ref[t] += float(wts[t, j]) * P.gated_expert(h[t:t + 1].double(), W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"])[0]
    # gate and up rows in turn in groups of 8, and all gate rows before all up rows
    stacked = torch.cat([gate.view(experts, F // 8, 8, D), up.view(experts, F // 8, 8, D)], dim=2).reshape(experts, 2 * F, D).contiguous().to(DEV)
    halves = torch.cat([gate, up], dim=1).contiguous().to(DEV)
    mid = torch.zeros(T * top, F, dtype=td, device=DEV)
    y = torch.full((T, D), 5.0, device=DEV)
    ops.moe_experts(h.to(DEV), stacked, down.to(DEV), ids, wts, mid, y, ops.ACT_SILU, gated=ops.GATED_GROUPS_OF_8)
    assert_close(to_np(y), ref.numpy(), dtype, "a warp per output")
    ops.moe_experts(h.to(DEV), halves, down.to(DEV), ids, wts, mid, y, ops.ACT_SILU, accumulate=True, gated=ops.GATED_HALVES)
    assert_close(to_np(y), 2 * ref.numpy(), dtype, "added, the other layout")
    if dtype == "bfloat16":
        take = lambda shape, dt: torch.empty(shape, dtype=dt, device=DEV)       # noqa: E731
        assert ops.moe_grouped_ok(h.to(DEV), stacked, ops.GATED_GROUPS_OF_8) and not ops.moe_grouped_ok(h.to(DEV), halves, ops.GATED_HALVES)
        y2 = torch.full((T, D), 5.0, device=DEV)
        ops.moe_experts_grouped(h.to(DEV), stacked, down.to(DEV), ids, wts, y2, ops.ACT_SILU, False, take, gated=ops.GATED_GROUPS_OF_8)
        assert_close(to_np(y2), ref.numpy(), dtype, "grouped by expert")
        assert not ops.moe_tc_ok(h.to(DEV), stacked, top, ops.GATED_GROUPS_OF_8, ops.ACT_SILU) or T * top >= 512
        y3 = torch.full((T, D), 5.0, device=DEV)
        ops.moe_experts_tc(h.to(DEV), stacked, down.to(DEV), ids, wts, y3, False, take)
        torch.cuda.synchronize()
        ops.check_kernel_errors()
        assert_close(to_np(y3), ref.numpy(), dtype, "grouped by expert, tcgen05")
        ops.moe_experts_tc(h.to(DEV), stacked, down.to(DEV), ids, wts, y3, True, take)
        assert_close(to_np(y3), 2 * ref.numpy(), dtype, "grouped by expert, tcgen05, added")


class _Cache:
    """A paged cache of one plane filled from keys [L, G, d] of one sequence, its pages out of order."""

    def __init__(self, keys, td, page=64, spare=3):
        L, G, d = keys.shape
        n = -(-L // page)
        order = torch.randperm(n + spare, generator=torch.Generator().manual_seed(L))[:n]
        self.k = torch.zeros(n + spare, G, page, d, dtype=td, device=DEV)
        for j in range(L):
            self.k[int(order[j // page]), :, j % page] = keys[j].to(td).to(DEV)
        self.pages = order.to(torch.int32).view(1, n).to(DEV)
        self.page = page


def _attend(kernel, q, cache, pos0, H, G, d, scale, cap, sink, td):
    """Queries q [n, H, d] at positions pos0.. over the cache, through one of the kernels."""
    n = q.shape[0]
    qd = q.reshape(n, H * d).to(td).to(DEV).contiguous()
    out = torch.zeros(n, H * d, dtype=td, device=DEV)
    sk = None if sink is None else sink.float().to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)       # noqa: E731
    if kernel == "simt":
        ops.attention_simt(qd, H * d, out, cache.k, cache.k, i32([0] * n), i32(list(range(pos0, pos0 + n))), cache.pages,
                           H, G, d, cache.page, scale, None, cap, sk)
    elif kernel == "decode":
        assert n == 1
        for nsplit in (1, 3):
            buf = torch.zeros(ops.attention_decode_scratch_floats(1, H, d, nsplit), device=DEV)
            ops.attention_decode(qd, H * d, out, cache.k, cache.k, i32([pos0 + 1]), cache.pages, buf, H, G, d, cache.page,
                                 min(nsplit, cache.pages.shape[1]), scale, None, cap, sk)
            if nsplit == 1:
                first = out.clone()
        assert float((out.float() - first.float()).abs().max()) <= 2e-2 * float(first.float().abs().max())
    else:
        fn = ops.attention_prefill_tc if kernel == "prefill_tc" else ops.attention_prefill
        fn(qd, H * d, out, cache.k, cache.k, i32([0, n]), i32([pos0]), cache.pages, 1, n, H, G, d, cache.page, scale, None, cap, sk)
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    return to_np(out).reshape(n, H, d)


KERNELS = [("float32", "simt", 24), ("bfloat16", "simt", 24), ("bfloat16", "decode", 32), ("bfloat16", "decode", 64),
           ("bfloat16", "decode", 128), ("bfloat16", "decode", 80), ("bfloat16", "prefill", 32), ("bfloat16", "prefill", 80),
           ("bfloat16", "prefill_tc", 64), ("bfloat16", "prefill_tc", 128)]


@pytest.mark.parametrize("dtype,kernel,d", KERNELS)
def test_attention_kernels_on_a_crafted_cache(dtype, kernel, d):
    """One key carries the softmax of a query: far back among hundreds, at a page's last and first place,
    the very first, the query's own.  Then a sink that takes most of the weight, and two keys beyond the cap
    (equal after it, far apart before it).  Values are the keys: the result is read off the key itself."""
    td = td_of(dtype)
    g = torch.Generator().manual_seed(d)
    H, G, L = 4, 2, 700
    keys = (torch.randn(L, G, d, generator=g) * 0.3).to(torch.bfloat16).double()
    scale = 1.0 / math.sqrt(d)
    cache = _Cache(keys, td)
    one = kernel == "decode"
    for target in (3, 63, 64, 0, 447, 448, 699):
        # the last query (position 699) looks for `target`; in a prompt's portion the queries before it do too
        n = 1 if one else 150
        q = torch.randn(n, H, d, generator=g, dtype=torch.float64) * 0.3
        for i in range(H):
            q[:, i] += keys[target, i // 2] * (12.0 / scale / float(keys[target, i // 2] @ keys[target, i // 2]))
        q = q.to(torch.bfloat16).double()
        ref = P.attention_heads(torch.cat([torch.zeros(L - n, H, d, dtype=torch.float64), q]), keys, keys, scale, 30.0, None)[L - n:]
        rows = [r for r in range(n) if L - n + r >= target]
        assert float((ref[rows[-1]] - keys[target].repeat_interleave(2, 0)).abs().max()) < 0.3 * float(keys[target].abs().max())
        got = _attend(kernel, q, cache, L - n, H, G, d, scale, 30.0, None, td)
        assert_close(got[rows], ref[rows].numpy(), dtype, f"{kernel} key {target}")
    # a sink that outweighs the keys for heads 0 and 3, and is negligible for the others
    n = 1 if one else 70
    q = (torch.randn(n, H, d, generator=g, dtype=torch.float64)).to(torch.bfloat16).double()
    sink = torch.tensor([8.0, -20.0, 0.5, 9.0], dtype=torch.float64)
    ref = P.attention_heads(torch.cat([torch.zeros(L - n, H, d, dtype=torch.float64), q]), keys, keys, scale, None, sink)[L - n:]
    bare = P.attention_heads(torch.cat([torch.zeros(L - n, H, d, dtype=torch.float64), q]), keys, keys, scale, None, None)[L - n:]
    assert float(ref[:, 0].abs().max()) < 0.6 * float(bare[:, 0].abs().max())
    got = _attend(kernel, q, cache, L - n, H, G, d, scale, None, sink, td)
    assert_close(got, ref.numpy(), dtype, f"{kernel} sink")
    # the first tokens of a sequence: the sink beside one, two, three keys
    short = _Cache(keys[:5], td)
    for pos in ([0, 1, 4] if one else [0]):
        m = 1 if one else 5
        q = (torch.randn(m, H, d, generator=g, dtype=torch.float64) * 2).to(torch.bfloat16).double()
        pad = torch.zeros(pos, H, d, dtype=torch.float64)
        ref = P.attention_heads(torch.cat([pad, q]), keys[:pos + m], keys[:pos + m], scale, 5.0, sink)[pos:]
        got = _attend(kernel, q, short, pos, H, G, d, scale, 5.0, sink, td)
        assert_close(got, ref.numpy(), dtype, f"{kernel} first tokens from {pos}")
    # two keys beyond the cap
    n = 1 if one else 40
    q = torch.randn(n, H, d, generator=g, dtype=torch.float64) * 0.2
    a, b = 100, 650
    for i in range(H):
        ka, kb = keys[a, i // 2], keys[b, i // 2]
        q[:, i] += ka * (14.0 / scale / float(ka @ ka)) + kb * (40.0 / scale / float(kb @ kb))
    q = q.to(torch.bfloat16).double()
    ref = P.attention_heads(torch.cat([torch.zeros(L - n, H, d, dtype=torch.float64), q]), keys, keys, scale, 4.0, sink)[L - n:]
    uncapped = P.attention_heads(torch.cat([torch.zeros(L - n, H, d, dtype=torch.float64), q]), keys, keys, scale, None, sink)[L - n:]
    assert float((ref - uncapped).abs().max()) > 0.2 * float(ref.abs().max())
    got = _attend(kernel, q, cache, L - n, H, G, d, scale, 4.0, sink, td)
    assert_close(got, ref.numpy(), dtype, f"{kernel} cap")


# ---- whole models -----------------------------------------------------------------------------------
ALONE = {
    "attention": [(U.attention(sharp=3.0), None)],
    "attention_plain": [(U.attention(softcap=None, coef=None, heads=2, kv_heads=2), None)],
    "attention_64": [(U.attention(heads=4, kv_heads=1, dim=64, every=2), None)],
    "moe": [(U.attention(heads=1, kv_heads=1, dim=8), U.moe())],
    "moe_no_groups_no_shared": [(U.attention(heads=1, kv_heads=1, dim=8), U.moe(groups=None, shared=None, top=3))],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", sorted(ALONE))
def test_one_layer_of_each_kind(tmp_path, which, dtype):
    d, pm = U.make(tmp_path / which, ALONE[which], seed=len(which))
    ids = ids_for(np.random.default_rng(1), 131, 70)
    eng = engine_for(d, dtype, max_tokens=512)
    ref = pm.logits(ids).numpy()
    assert_close(replay_whole(eng, ids), ref, dtype, which, plain=pm, ids=ids)
    assert_close(replay_tail_one_by_one(eng, ids, 69), ref, dtype, which + " token by token", plain=pm, ids=ids)


def test_the_residual_stream_after_every_layer(mixed):
    d, pm = mixed
    ids = ids_for(np.random.default_rng(4), 131, 33)
    want = []
    pm.hidden(ids, layers_out=want)
    eng = engine_for(d, "float32", max_tokens=256)
    got = []
    for b in eng.model.blocks:
        def run(x, batch, cache, inner=b.forward, **kw):
            out = inner(x, batch, cache, **kw)
            got.append(to_np(x))
            return out
        b.forward = run
    replay_whole(eng, ids)
    assert len(got) == len(want) == 4
    for i, (a, b) in enumerate(zip(got, want)):
        assert np.abs(a - b.numpy()).max() < 3e-5 * float(b.abs().max()), i


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_against_token_by_token_and_pieces(mixed, dtype):
    d, pm = mixed
    ids = ids_for(np.random.default_rng(2), 131, 90)
    ref = pm.logits(ids).numpy()
    eng = engine_for(d, dtype, max_tokens=1024)
    assert_close(replay_whole(eng, ids), ref, dtype, "whole", plain=pm, ids=ids)
    assert_close(replay_tail_one_by_one(eng, ids, 89), ref, dtype, "one by one", plain=pm, ids=ids)
    for piece in (2, 3, 16, 21, 64):
        s, rows = eng.alloc_slot(), []
        for at in range(0, len(ids), piece):
            rows.append(to_np(eng.step([(s, ids[at:at + piece])], "all")))
        eng.free_slot(s)
        assert_close(np.concatenate(rows), ref, dtype, f"pieces of {piece}", plain=pm, ids=ids)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batches_in_slots_and_pages_that_were_used_before(mixed, dtype):
    d, pm = mixed
    rng = np.random.default_rng(3)
    reqs = [ids_for(rng, 131, n) for n in (1, 37, 80, 5, 64, 23, 2, 70)]
    refs = [pm.logits(r).numpy() for r in reqs]
    eng = engine_for(d, dtype, max_tokens=64 * 5, max_slots=3)          # every slot and page is handed out again
    got = replay_batches(eng, reqs, [1, 30, 64, 2, 40, 23, 1, 65], [[0, 1, 2], [3, 4], [5, 6, 7]])
    for i, (g, ref) in enumerate(zip(got, refs)):
        assert_close(g, ref, dtype, f"request {i}", plain=pm, ids=reqs[i])
    assert eng.cache.slots.free_count == 3


@pytest.mark.parametrize("dtype", DTYPES)
def test_sharp_attention_over_small_pages_and_long_decoding(tmp_path, dtype):
    """Sharp attention (a few keys carry the softmax) with a temperature that steps every third position,
    pages of 16: the prompt whole, and 170 tokens decoded one by one across ten page borders."""
    layers = [(U.attention(heads=2, kv_heads=1, dim=16, sharp=4.0, every=3), U.moe()),
              (U.attention(heads=2, kv_heads=2, dim=64, sharp=4.0, every=3, softcap=4.0), None)]
    d, pm = U.make(tmp_path / "s", layers, seed=11)
    ids = ids_for(np.random.default_rng(11), 131, 220)
    ref = pm.logits(ids).numpy()
    page = 16 if dtype == "float32" else 64       # the tensor-core kernels read pages in tiles of 64 keys
    eng = engine_for(d, dtype, max_tokens=page * 16, page_size=page)
    bound = sensitivity_bound(pm, ids, dtype)
    assert_close(replay_whole(eng, ids), ref, dtype, "whole", bound=bound)
    assert_close(replay_tail_one_by_one(eng, ids, 170), ref, dtype, "decoded", bound=bound)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_long_prompt_and_its_continuation(tmp_path, dtype):
    """600 tokens at once (several tiles of pairs per expert, ten pages of keys, the temperature far along), then the
    same prompt in two portions and 24 tokens decoded one by one."""
    layers = [(U.attention(heads=4, kv_heads=2, dim=32, every=100, softcap=15.0), U.moe(experts=8, top=2, groups=4, keep=2, ff=48, shared=72)),
              (U.attention(heads=2, kv_heads=1, dim=64, every=100, coef=0.2), U.moe(experts=8, top=2, groups=4, keep=2, ff=48, shared=72))]
    d, pm = U.make(tmp_path / "long", layers, seed=13, width=128, vocab=500, max_positions=1024)
    ids = ids_for(np.random.default_rng(13), 500, 624)
    rows = [0, 1, 63, 64, 99, 100, 299, 300, 511, 512, 598, 599] + list(range(600, 624))
    arith = torch.float32 if dtype == "bfloat16" else torch.float64
    ref = pm.logits(ids).numpy()[rows]
    eng = engine_for(d, dtype, max_tokens=2048)
    for cuts in ([600], [333, 267]):
        s, got, at = eng.alloc_slot(), [], 0
        for n in cuts + [1] * 24:
            want = [r - at for r in rows if at <= r < at + n]
            out = eng.step([(s, ids[at:at + n])], [want])
            if want:
                got.append(to_np(out))
            at += n
        eng.free_slot(s)
        assert_close(np.concatenate(got), ref, dtype, f"prompt in {len(cuts)}", plain=pm, ids=ids, rows=rows, arith=arith)
    eng.check_kernels()


def test_a_temperature_period_one_off_shows(tmp_path):
    """The comparison is sharp enough to see a period that is one position too long or too short."""
    d, pm = U.make(tmp_path / "t", [(U.attention(every=9, coef=0.8, sharp=2.0), None)], seed=1)
    ids = ids_for(np.random.default_rng(0), 131, 60)
    got = replay_whole(engine_for(d, "float32", max_tokens=256), ids)
    for off in (8, 10):
        cfg = dict(pm.cfg, layers=[dict(pm.cfg["layers"][0], mixer=dict(pm.cfg["layers"][0]["mixer"], q_temp={"coef": 0.8, "every": off}))])
        wrong = P.PlainVotapel(config=cfg, tensors=pm.w).logits(ids).numpy()
        assert np.abs(got - wrong).max() > 1e-2
    assert np.abs(got - pm.logits(ids).numpy()).max() < 1e-4


OTHER = {
    "one_head_top_one": ([(U.attention(heads=1, kv_heads=1, dim=8, every=1), U.moe(experts=2, top=1, groups=2, keep=1, ff=8, shared=8, scale=1.0)),
                          (U.attention(heads=1, kv_heads=1, dim=8, coef=None), None)], dict(vocab=77, width=40, mult=1.0, eps=1e-6)),
    "wide_heads": ([(U.attention(heads=6, kv_heads=2, dim=96, every=40), U.moe(experts=9, top=6, groups=3, keep=2, ff=40, shared=None)),
                    (U.attention(heads=5, kv_heads=5, dim=48, softcap=50.0), U.moe(experts=9, top=6, groups=3, keep=2, ff=72, shared=136))],
                   dict(vocab=300, width=136, mult=0.3)),
    "odd_sizes": ([(U.attention(heads=3, kv_heads=1, dim=10, every=4), U.moe(experts=3, top=3, groups=1, keep=1, ff=12, shared=30)),
                   (U.attention(heads=6, kv_heads=3, dim=20), U.moe(experts=3, top=3, groups=1, keep=1, ff=20, shared=6))],
                  dict(vocab=61, width=50, mult=1.4)),
    "many_experts": ([(U.attention(heads=8, kv_heads=8, dim=32), U.moe(experts=32, top=4, groups=8, keep=3, ff=16, shared=16, scale=2.5)),
                      (U.attention(heads=2, kv_heads=1, dim=160), U.moe(experts=32, top=4, groups=8, keep=3, ff=16, shared=16, scale=2.5))],
                     dict(vocab=200, width=128)),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", sorted(OTHER))
def test_other_sizes_and_orders(tmp_path, which, dtype):
    layers, kw = OTHER[which]
    d, pm = U.make(tmp_path / which, layers, seed=7, **kw)
    rng = np.random.default_rng(5)
    reqs = [ids_for(rng, kw["vocab"], n) for n in (130, 2, 66)]
    refs = [pm.logits(r).numpy() for r in reqs]
    eng = engine_for(d, dtype, max_tokens=64 * 8, max_slots=3)
    assert_close(replay_whole(eng, reqs[0]), refs[0], dtype, "whole", plain=pm, ids=reqs[0])
    assert_close(replay_tail_one_by_one(eng, reqs[0], 40), refs[0], dtype, "tail", plain=pm, ids=reqs[0])
    got = replay_batches(eng, reqs, [100, 1, 30], [[0, 1, 2]])
    for g, ref, r in zip(got, refs, reqs):
        assert_close(g, ref, dtype, "batched", plain=pm, ids=r)


def test_a_router_without_help_in_32_bit(tmp_path):
    """Random routers (no decisive channels), layers with different feed-forward shapes: in 32-bit the
    choice is the plain model's everywhere."""
    d, pm = U.make(tmp_path / "r", [(U.attention(), U.moe(experts=8, top=3, groups=4, keep=2)),
                                    (U.attention(), U.moe(experts=6, top=2, groups=2, keep=1, shared=None))], seed=9,
                   decisive_router=False)
    ids = ids_for(np.random.default_rng(9), 131, 120)
    eng = engine_for(d, "float32", max_tokens=512)
    ref = pm.logits(ids).numpy()
    assert_close(replay_whole(eng, ids), ref, "float32", "whole")
    assert_close(replay_tail_one_by_one(eng, ids, 30), ref, "float32", "tail")


def test_a_sequence_cannot_outgrow_the_position_table(tmp_path):
    d, pm = U.make(tmp_path / "p", [(U.attention(), None)], seed=2, max_positions=40)
    eng = engine_for(d, "float32", max_tokens=256)
    s = eng.alloc_slot()
    eng.step([(s, list(range(40)))], "last")
    with pytest.raises(hb.errors.HerbertError):
        eng.step([(s, [1])], "last")
    eng.free_slot(s)


@pytest.mark.parametrize("dtype", DTYPES)
def test_captured_decode_steps_equal_eager_ones(mixed, dtype):
    d, pm = mixed
    rng = np.random.default_rng(8)
    reqs = [ids_for(rng, 131, n) for n in (40, 70)]
    out = []
    for graphs in (True, False):
        eng = engine_for(d, dtype, max_tokens=1024, use_graphs=graphs)
        out.append(replay_batches(eng, reqs, [10, 33], [[0, 1]]))
        if graphs:
            assert eng.graph_replays > 20
    for a, b in zip(*out):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_any_shape_attention_kernel_agrees_with_the_tensor_core_ones(mixed, dtype):
    d, pm = mixed
    ids = ids_for(np.random.default_rng(12), 131, 100)
    ref = pm.logits(ids).numpy()
    ops.options.attention = "simt"
    try:
        eng = engine_for(d, dtype, max_tokens=512)
        assert_close(replay_tail_one_by_one(eng, ids, 20), ref, dtype, "simt", plain=pm, ids=ids)
    finally:
        ops.options.attention = "auto"


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(mixed, dtype):
    d, pm = mixed
    eng = engine_for(d, dtype, max_tokens=2048)
    rng = np.random.default_rng(15)
    prompts = [ids_for(rng, 131, n) for n in (9, 1, 30, 4, 17)]
    res = hb.generate(eng, prompts, hb.GenerationOptions(max_tokens=10, ignore_eos=True, max_batch=3),
                      hb.SamplingParams(temperature=0.0))
    assert res.stats.batches == 2 and all(len(t) == 10 for t in res.tokens)
    for p, got in zip(prompts, res.tokens):
        ids = list(p)
        for tok in got:
            ref = pm.logits(ids)[-1].numpy()
            margin = 1e-4 if dtype == "float32" else 2 * bound_for(pm, ids, dtype, ref, rows=[len(ids) - 1])
            assert ref.max() - ref[tok] <= margin
            ids.append(tok)
    eng.cache.check()
    assert eng.cache.slots.free_count == eng.cache.num_slots


def test_random_weights_from_the_configuration(tmp_path):
    cfg = U.config([(U.attention(), U.moe()), (U.attention(heads=2, kv_heads=2, dim=32), None)])
    hb.write_random_model(cfg, str(tmp_path), seed=1)
    pm = P.PlainVotapel(str(tmp_path))
    assert pm.w["pos"].shape == (512, 64) and float(pm.w["l0.norm1"].abs().max()) < 0.6       # norm weights around zero
    ids = ids_for(np.random.default_rng(1), 131, 50)
    eng = engine_for(str(tmp_path), "float32", max_tokens=256)
    assert_close(replay_whole(eng, ids), pm.logits(ids).numpy(), "float32", "random model")


def test_command_line_trace_replay_and_prompts_in_pieces(mixed, tmp_path, capsys):
    """The design through the library's other entry points: the command line, `bin/trace_run`, and the
    generation loop with prompts fed in pieces and sampling on the device."""
    import json
    import os
    import subprocess
    import sys
    from herbert_rs_b200 import cli
    d, pm = mixed
    rng = np.random.default_rng(21)
    a, b = ids_for(rng, 131, 40), ids_for(rng, 131, 7)
    assert cli.main(["--model", d, "--prompt-ids", ",".join(map(str, a)), "--prompt-ids", ",".join(map(str, b)),
                     "--max-tokens", "5", "--temperature", "0", "--ignore-eos", "--backend", "cuda-fp32"]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    assert len(lines) == 2
    ids = list(a)
    for tok in map(int, lines[0].split(",")):
        ref = pm.logits(ids)[-1].numpy()
        assert ref.max() - ref[tok] <= 1e-4
        ids.append(tok)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}, {"id": "b", "tokens": b[:6], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]}, {"id": "b", "tokens": b[6:], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[31:32], "want": [0]}], "end": ["a"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype in DTYPES:
        out = tmp_path / ("trace_" + dtype)
        r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True)
        assert r.returncode == 0 and [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
        ra, rb = pm.logits(a).numpy(), pm.logits(b).numpy()
        read = lambda n, rows: np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(rows, 131).astype(np.float64)      # noqa: E731
        assert_close(read(0, 2), ra[[0, 29]], dtype, "trace step 0", plain=pm, ids=a, rows=[0, 29])
        assert_close(read(1, 2)[:1], ra[[30]], dtype, "trace step 1 a", plain=pm, ids=a, rows=[30])
        assert_close(read(1, 2)[1:], rb[[6]], dtype, "trace step 1 b", plain=pm, ids=b, rows=[6])
        assert_close(read(2, 1), ra[[31]], dtype, "trace step 2", plain=pm, ids=a, rows=[31])
    outs = []
    for piece in (None, 16):
        eng = engine_for(d, "float32", max_tokens=1024)
        res = hb.generate(eng, [a, b], hb.GenerationOptions(max_tokens=8, ignore_eos=True, prefill_chunk_size=piece),
                          hb.SamplingParams(temperature=0.8, top_k=20, top_p=0.95, seed=5))
        outs.append(res.tokens)
    assert outs[0] == outs[1]
