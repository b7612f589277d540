"""The Kebisun design in the engine against the plain implementation (`plain_kebisun.py`): every
mechanism alone, prompts against decoding, prompts in pieces, unequal batches, slots and pages that
are used again, window edges and page borders, long decoding, other sizes, greedy generation."""
import math

import numpy as np
import pytest
import torch

import herbert_rs_b200 as hb
import kebisun_util as K
import plain_kebisun as P
from gpu_util import (DTYPES, assert_close, engine_for, replay_batches, replay_tail_one_by_one, replay_whole,
                      sensitivity_bound, to_np)
from herbert_rs_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def ids_for(rng, cfg_or_vocab, n):
    v = cfg_or_vocab if isinstance(cfg_or_vocab, int) else cfg_or_vocab["vocab"]
    return rng.integers(0, v, n).tolist()


@pytest.fixture(scope="module")
def mixed(tmp_path_factory):
    """Both mixers, both feed-forwards, a layer without feed-forward; a window that is no multiple of anything."""
    layers = [(K.latent(window=21), K.dense()), (K.gla(), K.moe()), (K.latent(heads=2, vdim=16, window=21), None),
              (K.gla(heads=3, dim=16, vdim=24, tau=3.0), K.dense(ff=40)),
              (K.latent(window=21, kv_rank=64, rot=16), K.moe(experts=5, top=3, ff=16))]     # sizes the tensor-core kernel serves
    return K.make(tmp_path_factory.mktemp("kebisun_mixed"), layers, seed=3)


# ---- each mechanism alone -------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim", [48, 200, 1000])
def test_layer_norm_alone_and_with_the_scaled_residual_sum(dtype, dim):
    g = torch.Generator().manual_seed(dim)
    y = (torch.randn(7, dim, generator=g) * 3 + 1.5).to(DEV)
    x = torch.randn(7, dim, generator=g).to(DEV)
    w, s = (1 + 0.2 * torch.randn(dim, generator=g)).to(DEV), (1 + 0.2 * torch.randn(dim, generator=g)).to(DEV)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    out = torch.empty(3, dim, dtype=td, device=DEV)
    rows = torch.tensor([4, 0, 6], dtype=torch.int32, device=DEV)
    ops.layernorm(y, w, out, 1e-5, rows)
    ref = P.layer_norm(y.double().cpu()[[4, 0, 6]], w.double().cpu(), 1e-5)
    assert_close(to_np(out), ref.numpy(), dtype, "layernorm rows")
    x2, h = x.clone(), torch.empty(7, dim, dtype=td, device=DEV)
    ops.layernorm_residual(y, w, s, x2, h, 1e-5, td)
    ref = x.double().cpu() + P.layer_norm(y.double().cpu(), w.double().cpu(), 1e-5) * s.double().cpu()
    assert_close(to_np(x2), ref.numpy(), "float32", "residual sum")
    assert_close(to_np(h), ref.numpy(), dtype, "next input")
    x3 = x.clone()
    ops.layernorm_residual(y, w, None, x3, None, 1e-5, td)
    ref = x.double().cpu() + P.layer_norm(y.double().cpu(), w.double().cpu(), 1e-5)
    assert_close(to_np(x3), ref.numpy(), "float32", "without scale")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter,interleave", [(40, 8), (24, 0), (30, 0)])
@pytest.mark.parametrize("act", ["gelu_tanh", "gelu", "silu"])
def test_gated_activation_kernel(dtype, inter, interleave, act):
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(inter)
    gate, up = (torch.randn(9, inter, generator=g) * 2).to(td), torch.randn(9, inter, generator=g).to(td)
    if interleave:
        gu = torch.cat([gate.view(9, -1, 1, 8), up.view(9, -1, 1, 8)], dim=2).reshape(9, 2 * inter)
    else:
        gu = torch.cat([gate, up], dim=1)
    out = torch.empty(9, inter, dtype=td, device=DEV)
    ops.swiglu(gu.contiguous().to(DEV), out, interleave, ops.ACTIVATIONS[act])
    f = {"gelu_tanh": P.gelu_tanh, "gelu": P.gelu_erf, "silu": P.silu}[act]
    assert_close(to_np(out), (f(gate.double()) * up.double()).numpy(), dtype, act)


@pytest.mark.parametrize("scaling", [True, False])
def test_rotation_with_stretched_frequencies(scaling):
    from herbert_rs_b200.config.specs import ScaledRotarySpec
    from herbert_rs_b200.parts import ScaledRotary
    rot = {"base": 500.0, "dims": 12}
    spec = ScaledRotarySpec(12, 500.0)
    if scaling:
        rot["scaling"] = {"factor": 6.0, "original": 40, "fast": 6.0, "slow": 0.5}
        spec = ScaledRotarySpec(12, 500.0, 6.0, 40, 6.0, 0.5)
    part = ScaledRotary(spec, hb.Runtime(DEV, torch.float32))
    f, m = P.rotary_frequencies(rot, torch.float64)
    assert abs(part.mscale - m) < 1e-12 and np.allclose(part.freq.cpu().double().numpy(), f.numpy(), rtol=1e-7)
    if scaling:
        assert not np.allclose(f.numpy(), 500.0 ** (-2 * np.arange(6) / 12))      # some band is stretched
    g = torch.Generator().manual_seed(1)
    T, H, stride, off = 9, 3, 20, 8
    src = torch.randn(T, H * stride, generator=g).to(DEV)
    pos = torch.tensor([0, 1, 2, 63, 64, 65, 700, 5000, 12], dtype=torch.int32, device=DEV)
    out = torch.zeros(T, H * 14, device=DEV)
    ops.rotate_heads(src, stride, off, out, 14, 2, part.freq, part.mscale, pos, H, 12, scale=0.5)
    u = src.cpu().double().view(T, H, stride)[:, :, off:off + 12].transpose(0, 1)
    ref = (P.rotate(u, pos.cpu(), f, m) * 0.5).transpose(0, 1)
    got = to_np(out).reshape(T, H, 14)
    assert np.abs(got[:, :, 2:] - ref.numpy()).max() < 2e-4        # the angle itself is a float product
    assert np.abs(got[:, :, :2]).max() == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,K,N,stride", [(5, 3, 16, 40, 24), (70, 3, 16, 40, 24), (33, 2, 21, 10, 23), (130, 4, 72, 136, 80)])
def test_product_per_head(dtype, T, H, K, N, stride):
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(T + K)
    src = torch.randn(T, H * stride, generator=g)
    w = (torch.randn(H, N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    gate = torch.randn(T, H * N, generator=g)
    ref = torch.einsum("thk,hnk->thn", src.view(T, H, stride)[:, :, :K].double(), w.double()) * 0.7
    out = torch.zeros(T, H * (N + 3), device=DEV)
    ops.headwise_gemm(src.to(DEV), stride, w.to(td).to(DEV), out, N + 3, scale=0.7)
    got = to_np(out).reshape(T, H, N + 3)
    assert_close(got[:, :, :N], ref.numpy(), dtype, "into floats")
    assert np.abs(got[:, :, N:]).max() == 0.0
    out2 = torch.zeros(T, H * N, dtype=td, device=DEV)
    ops.headwise_gemm(src.to(DEV), stride, w.to(td).to(DEV), out2, N, scale=0.7, gate=gate.to(DEV))
    assert_close(to_np(out2).reshape(T, H, N), (ref * torch.sigmoid(gate.double()).view(T, H, N)).numpy(), dtype, "gated")


def _plain_latent_scores(q, rows, p, window, sink):
    """Softmax over rows lo..p with a sink, sum of the first `rank` numbers: float64, one query."""
    lo = max(0, p - window + 1) if window else 0
    s = rows[lo:p + 1] @ q
    top = max(float(s.max()), sink)
    e = torch.exp(s - top)
    return e / (e.sum() + math.exp(sink - top)), lo


class _Step:
    """The facts of a step that the tensor-core kernel reads: one sequence of `n` queries from position `p0`."""

    def __init__(self, n, p0):
        self.n_seqs, self.max_q_len = 1, n
        self.seq_start = torch.tensor([0, n], dtype=torch.int32, device=DEV)
        self.seq_pos0 = torch.tensor([p0], dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype,rank,rot,tensor_cores", [("float32", 24, 8, False), ("bfloat16", 24, 8, False),
                                                         ("bfloat16", 32, 16, True), ("bfloat16", 144, 16, True)])
def test_latent_attention_sees_exactly_its_window_also_across_pages(dtype, rank, rot, tensor_cores):
    """One cached row is made to stand out (its score is far above all others).  A query just inside
    the window must return that row's latent, a query one position further must not contain it: in a
    prompt's portion and for single decoded tokens, with the row at a page's last and first place, far
    back, and among the first tokens."""
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    H, page, window, n = 2, 16, 37, 200
    W = rank + rot
    tol = 2e-2 if tensor_cores else 2e-5                                      # there the weights are rounded to bfloat16
    g = torch.Generator().manual_seed(5)
    rows = torch.randn(n, W, generator=g) * 0.3
    pages_of_seq = torch.randperm(16, generator=g)[:13].to(torch.int32)       # scattered physical pages
    cache = torch.zeros(16, 1, page, W, dtype=td)
    for star in (0, 1, 15, 16, 17, 63, 64, 100, 150):
        rows_s = rows.clone()
        rows_s[star] = torch.randn(W, generator=g)
        rows_s = rows_s.to(td).double()
        for j in range(n):
            cache[pages_of_seq[j // page], 0, j % page] = rows_s[j].to(td)
        q1 = rows_s[star] * (12.0 / float(rows_s[star] @ rows_s[star]))       # score 12 at the star
        if tensor_cores:
            q1 = q1.to(torch.bfloat16).double()                               # the kernel's own rounding of the query
        for p_in in (star, star + 1, star + window - 1):                      # the star is seen ...
            for p in (p_in, star + window):                                    # ... and just not seen any more
                if p >= n:
                    continue
                q = torch.stack([q1, -q1]).reshape(1, H * W).float().to(DEV)
                out = torch.zeros(1, H * rank, device=DEV)
                sink = torch.tensor([0.5, -1.0], device=DEV)
                ops.latent_attention(q, out, cache.to(DEV), sink, torch.zeros(1, dtype=torch.int32, device=DEV),
                                     torch.tensor([p], dtype=torch.int32, device=DEV),
                                     pages_of_seq.view(1, -1).to(DEV), H, rank, rot, page, window,
                                     batch=_Step(1, p) if tensor_cores else None)
                for h, qq, sk in ((0, q1, 0.5), (1, -q1, -1.0)):
                    pr, lo = _plain_latent_scores(qq, rows_s, p, window, sk)
                    ref = pr @ rows_s[lo:p + 1, :rank]
                    got = to_np(out)[0, h * rank:(h + 1) * rank]
                    assert np.abs(got - ref.numpy()).max() < tol, (star, p, h)
                    if h == 0:
                        weight = float(pr[star - lo]) if lo <= star <= p else 0.0
                        assert (weight > 0.9) == (p < star + window), (star, p)
    # a portion of a prompt: many queries at once equal the single ones
    pos = torch.arange(40, 120, dtype=torch.int32)
    qs = torch.randn(len(pos), H * W, generator=g)
    out = torch.zeros(len(pos), H * rank, device=DEV)
    if tensor_cores:
        qs = qs.to(torch.bfloat16).float()
    ops.latent_attention(qs.to(DEV), out, cache.to(DEV), None, torch.zeros(len(pos), dtype=torch.int32, device=DEV), pos.to(DEV),
                         pages_of_seq.view(1, -1).to(DEV), H, rank, rot, page, window, batch=_Step(len(pos), 40) if tensor_cores else None)
    for i in (0, 7, 24, 79):
        for h in range(H):
            pr, lo = _plain_latent_scores(qs[i, h * W:(h + 1) * W].double(), rows_s, int(pos[i]), window, -math.inf)
            ref = pr @ rows_s[lo:int(pos[i]) + 1, :rank]
            assert np.abs(to_np(out)[i, h * rank:(h + 1) * rank] - ref.numpy()).max() < tol


def test_the_recurrence_carries_its_state_between_calls_and_keeps_far_tokens():
    """The scan kernel against the plain loop: whole, cut at every kind of place, per slot; a key
    written at the first token is still read 300 tokens later when its channel does not decay."""
    H, dk, dv, T = 2, 20, 36, 300
    g = torch.Generator().manual_seed(2)
    proj = torch.randn(T, H * (2 * dk + dv), generator=g) * 0.5
    decay = torch.rand(T, H * dk, generator=g) * 0.3 + 0.7
    decay[:, 3] = 1.0                                     # head 0, channel 3 never forgets
    proj[1:, H * dk + 3] = 0.0                            # and only token 0 writes to it
    q = proj[:, :H * dk].double().view(T, H, dk) * dk ** -0.5
    k = proj[:, H * dk:2 * H * dk].double().view(T, H, dk)
    v = proj[:, 2 * H * dk:].double().view(T, H, dv)
    S, ref = torch.zeros(H, dk, dv, dtype=torch.float64), []
    for t in range(T):
        S = decay[t].double().view(H, dk, 1) * S + k[t][:, :, None] * v[t][:, None, :]
        ref.append(torch.einsum("hkv,hk->hv", S, q[t]).reshape(-1))
    ref = torch.stack(ref).numpy()
    far = (k[0, 0, 3] * v[0, 0] * q[T - 1, 0, 3]).abs().max()
    assert far > 1e-3                                     # the far term is there to be lost
    for cuts in ([T], [1, 1, 2, 95, 1, 200], [150, 150]):
        state = torch.zeros(3, H, dk, dv, device=DEV)
        state[0] = 7.0                                    # another sequence's slot is not touched
        got, at = [], 0
        for n in cuts:
            out = torch.zeros(n, H * dv, device=DEV)
            ops.gla_scan(proj[at:at + n].contiguous().to(DEV), 0, H * dk, 2 * H * dk, decay[at:at + n].contiguous().to(DEV), state,
                         torch.tensor([2], dtype=torch.int32, device=DEV), torch.tensor([0, n], dtype=torch.int32, device=DEV),
                         out, 1, H, dk, dv, dk ** -0.5)
            got.append(to_np(out)); at += n
        assert np.abs(np.concatenate(got) - ref).max() < 3e-5 * np.abs(ref).max(), cuts
        assert float(state[0].min()) == 7.0 and float(state[1].abs().max()) == 0.0
        assert np.abs(to_np(state[2]) - S.numpy()).max() < 3e-5 * float(S.abs().max())


@pytest.mark.parametrize("tau", [1.0, 16.0])
def test_decays(tau):
    g = torch.Generator().manual_seed(4)
    low = torch.randn(11, 5, generator=g) * 3
    w2 = (torch.randn(14, 5, generator=g) * 2).to(torch.bfloat16).float()
    b = torch.randn(14, generator=g) * 2
    out = torch.zeros(11, 14, device=DEV)
    ops.gla_decay(low.to(DEV), w2.to(DEV), b.to(DEV), tau, out)
    ref = torch.sigmoid(low.double() @ w2.double().T + b.double()) ** (1.0 / tau)
    assert np.abs(to_np(out) - ref.numpy()).max() < 2e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top", [(5, 2), (1, 1), (40, 40), (33, 7)])
def test_router_and_experts(dtype, experts, top):
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(experts)
    T, D, F = 19, 48, 20
    h = torch.randn(T, D, generator=g).to(td)
    r = (torch.randn(experts, D, generator=g) * 0.5).to(torch.bfloat16).to(td)
    up = (torch.randn(experts, F, D, generator=g) / math.sqrt(D)).to(torch.bfloat16).to(td)
    down = (torch.randn(experts, D, F, generator=g) / math.sqrt(F)).to(torch.bfloat16).to(td)
    ids = torch.zeros(T, top, dtype=torch.int32, device=DEV)
    wts = torch.zeros(T, top, device=DEV)
    ops.moe_route(h.to(DEV), r.to(DEV), ids, wts, top)
    s = torch.softmax(h.double() @ r.double().T, -1)
    rw, ri = torch.topk(s, top, -1)
    assert (ids.cpu().long() == ri).all() and np.abs(to_np(wts) - rw.numpy()).max() < 1e-6
    if top < experts:
        assert float(wts.sum(-1).max()) < 1.0                       # not renormalized
    mid = torch.zeros(T * top, F, dtype=td, device=DEV)
    y = torch.full((T, D), 5.0, device=DEV)
    ops.moe_experts(h.to(DEV), up.to(DEV), down.to(DEV), ids, wts, mid, y, ops.ACT_GELU)
    W = {"router": r.double()}
    for e in range(experts):
        W[f"e{e}.up"], W[f"e{e}.down"] = up[e].double(), down[e].double()
    ref = P.routed_ff(h.double(), W, {"router": {"experts": experts, "top": top}})
    assert_close(to_np(y), ref.numpy(), dtype, "experts")


# ---- whole models -----------------------------------------------------------------------------------
ALONE = {
    "latent": [(K.latent(sharp=3.0), None)],
    "latent_plain_rotation": [(K.latent(scaling=False, window=7), None)],
    "gla": [(K.gla(), None)],
    "dense": [(K.gla(heads=1, dim=8, vdim=8), K.dense())],
    "moe": [(K.gla(heads=1, dim=8, vdim=8), K.moe())],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", sorted(ALONE))
def test_one_layer_of_each_kind(tmp_path, which, dtype):
    d, pm = K.make(tmp_path / which, ALONE[which], seed=len(which))
    rng = np.random.default_rng(1)
    ids = ids_for(rng, 131, 70)
    eng = engine_for(d, dtype, max_tokens=512)
    ref = pm.logits(ids).numpy()
    assert_close(replay_whole(eng, ids), ref, dtype, which, plain=pm, ids=ids)
    assert_close(replay_tail_one_by_one(eng, ids, 69), ref, dtype, which + " token by token", plain=pm, ids=ids)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_against_token_by_token_and_pieces(mixed, dtype):
    d, pm = mixed
    rng = np.random.default_rng(2)
    ids = ids_for(rng, 131, 90)
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
@pytest.mark.parametrize("window", [1, 16, 17, 40])
def test_window_edges_pages_and_long_decoding(tmp_path, dtype, window):
    """Sharp attention (a few keys carry the softmax), pages of 16 positions, windows of one, a page,
    a page and one: the prompt as a whole, and 150 tokens decoded one by one, while pages the window
    left are given back and used again."""
    layers = [(K.latent(window=window, sharp=4.0, heads=2), K.dense()),
              (K.latent(window=window, sharp=4.0, kv_rank=32, rot=16), None)]           # the second on the tensor cores in bfloat16
    d, pm = K.make(tmp_path / "w", layers, seed=window)
    rng = np.random.default_rng(window)
    ids = ids_for(rng, 131, 200)
    ref = pm.logits(ids).numpy()
    eng = engine_for(d, dtype, max_tokens=16 * 16, page_size=16)
    bound = sensitivity_bound(pm, ids, dtype)           # sharp on purpose: the bound follows from the model in 32-bit too
    assert_close(replay_whole(eng, ids), ref, dtype, "whole", bound=bound)
    assert_close(replay_tail_one_by_one(eng, ids, 150), ref, dtype, "decoded", bound=bound)
    if window <= 17:
        s = eng.alloc_slot()
        eng.step([(s, ids[:100])], "none")
        held = [p for p in eng.cache.pages_of(s, 0) if p >= 0]
        assert len(held) <= 2 + window // 16                           # the rest went back to the pool
        eng.free_slot(s)
    eng.cache.check()


def test_a_window_one_token_off_shows(tmp_path):
    """The comparison is sharp enough to see a window that is one token too long or too short."""
    d, pm = K.make(tmp_path / "w", [(K.latent(window=9, sharp=4.0), None)], seed=1)
    ids = ids_for(np.random.default_rng(0), 131, 60)
    got = replay_whole(engine_for(d, "float32", max_tokens=256), ids)
    for off in (8, 10):
        cfg = dict(pm.c, layers=[dict(pm.c["layers"][0], mixer=dict(pm.c["layers"][0]["mixer"], mask={"size": off}))])
        wrong = P.PlainKebisun(config=cfg, tensors=pm.w).logits(ids).numpy()
        assert np.abs(got - wrong).max() > 1e-2
    assert np.abs(got - pm.logits(ids).numpy()).max() < 1e-4


OTHER = {
    "one_head_top_one": [(K.latent(heads=1, dim=8, rot=2, vdim=8, kv_rank=8, q_rank=8, window=5), K.moe(experts=2, top=1, ff=8)),
                         (K.gla(heads=1, dim=8, vdim=8, tau=1.0), None)],
    "wide_heads": [(K.gla(heads=2, dim=72, vdim=100), K.moe(experts=9, top=9, ff=40)),
                   (K.latent(heads=5, dim=40, rot=24, vdim=48, kv_rank=136, q_rank=72, window=100), K.dense(ff=200))],
    "gla_only": [(K.gla(), K.dense()), (K.gla(heads=4, dim=130, vdim=33), K.dense()), (K.gla(heads=1, dim=300, vdim=20), None)],
    "odd_sizes": [(K.latent(heads=3, dim=10, rot=6, vdim=6, kv_rank=20, q_rank=14, window=33), K.dense(ff=30)),
                  (K.gla(heads=3, dim=10, vdim=14, tau=5.0), K.moe(experts=3, top=2, ff=12))],
    "latent_only": [(K.latent(rot=16, dim=8), K.moe()), (K.latent(kv_rank=16, vdim=72, window=300), K.moe())],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", sorted(OTHER))
def test_other_sizes_and_orders(tmp_path, which, dtype):
    kw = dict(vocab=77, width=40, emb_scale=1.0, eps=1e-6) if which == "one_head_top_one" else \
        dict(vocab=61, width=50) if which == "odd_sizes" else dict(vocab=300, width=136)
    d, pm = K.make(tmp_path / which, OTHER[which], seed=7, decay_rank=3 if which in ("gla_only", "odd_sizes") else 16, **kw)
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
    """Random routers (no decisive channels): in 32-bit the choice is the plain model's everywhere."""
    d, pm = K.make(tmp_path / "r", [(K.latent(), K.moe(experts=7, top=3)), (K.gla(), K.moe(experts=4, top=2))], seed=9,
                   decisive_router=False)
    ids = ids_for(np.random.default_rng(9), 131, 120)
    eng = engine_for(d, "float32", max_tokens=512)
    ref = pm.logits(ids).numpy()
    assert_close(replay_whole(eng, ids), ref, "float32", "whole")
    assert_close(replay_tail_one_by_one(eng, ids, 30), ref, "float32", "tail")


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
def test_greedy_generation_through_the_entry_point(mixed, dtype):
    d, pm = mixed
    eng = engine_for(d, dtype, max_tokens=2048)
    rng = np.random.default_rng(15)
    prompts = [ids_for(rng, 131, n) for n in (9, 1, 30, 4, 17)]
    res = hb.generate(eng, prompts, hb.GenerationOptions(max_tokens=10, ignore_eos=True, max_batch=3),
                      hb.SamplingParams(temperature=0.0))
    assert res.stats.batches == 2 and all(len(t) == 10 for t in res.tokens)
    from gpu_util import bound_for
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
    """`write_random_model` serves the design too (the decay's inner size is then the configuration's
    optional "decay_rank", else a default), and the engine runs what it wrote."""
    cfg = K.config([(K.latent(), K.moe()), (K.gla(), K.dense())])
    cfg["layers"][1]["mixer"]["decay_rank"] = 5
    hb.write_random_model(cfg, str(tmp_path), seed=1)
    pm = P.PlainKebisun(str(tmp_path))
    assert pm.w["l1.mix.a1"].shape == (5, 64)
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
    # trace replay: a prompt in two steps, a second request joining as a batch of its own
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:], "want": [9]}], "end": ["a"]},
             {"step": 2, "entries": [{"id": "b", "tokens": b, "want": list(range(7))}], "end": ["b"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "trace"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True)
    assert r.returncode == 0 and [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    ra, rb = pm.logits(a).numpy(), pm.logits(b).numpy()
    assert_close(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, 131).astype(np.float64), ra[[0, 29]], "float32", "trace step 0")
    assert_close(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, 131).astype(np.float64), ra[[39]], "float32", "trace step 1")
    assert_close(np.fromfile(out / "2.f32", dtype="<f4").reshape(7, 131).astype(np.float64), rb, "float32", "trace step 2")
    # generation with prompts in pieces of 16 and sampling: the same tokens as with whole prompts
    outs = []
    for piece in (None, 16):
        eng = engine_for(d, "float32", max_tokens=1024)
        res = hb.generate(eng, [a, b], hb.GenerationOptions(max_tokens=8, ignore_eos=True, prefill_chunk_size=piece),
                          hb.SamplingParams(temperature=0.8, top_k=20, top_p=0.95, seed=5))
        outs.append(res.tokens)
    assert outs[0] == outs[1]
