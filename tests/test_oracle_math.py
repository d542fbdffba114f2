"""Self-consistency of the CPU oracle: its two evaluation modes, the tie rule,
absorbed against non-absorbed MLA, and independent numpy restatements."""
import numpy as np
import pytest

import util


def test_dequant_is_rounded_product(oracle):
    rng = np.random.default_rng(1)
    q, w = util.rand_i4(rng, 16, 128)
    s = util.rand_scales(rng, 16, 4)
    deq = oracle.i4_dequant(w, s)
    expect = util.f32_to_bf16_np(q.astype(np.float32) * np.repeat(util.bf16_np_to_f32(s), 32, axis=1))
    assert np.array_equal(deq, expect)


@pytest.mark.parametrize("rows,cols", [(1, 32), (5, 96), (64, 7168), (65, 2048)])
def test_i4_gemv_modes_agree(oracle, rows, cols):
    rng = np.random.default_rng(rows * 7 + cols)
    _, w = util.rand_i4(rng, rows, cols)
    s = util.rand_scales(rng, rows, cols // 32)
    x = oracle.bf16_round(rng.normal(size=cols).astype(np.float32))
    wide = oracle.i4_gemv(w, s, x, mode=0, round_out=False)
    exact = oracle.i4_gemv(w, s, x, mode=1, round_out=True)
    deq = util.bf16_np_to_f32(oracle.i4_dequant(w, s)).astype(np.float64)
    ref = deq @ x.astype(np.float64)
    np.testing.assert_allclose(wide, ref, rtol=1e-5, atol=1e-6)
    scale = np.max(np.abs(ref)) + 1e-30
    assert np.max(np.abs(exact - ref)) / scale < 1e-2  # one bf16 rounding of the output


def test_i4_gemv_empty(oracle):
    y = oracle.i4_gemv(np.zeros((0, 4), np.uint32), np.zeros((0, 1), np.uint16), np.zeros(32, np.float32))
    assert y.shape == (0,)


def test_router_tie_goes_to_lowest_index_and_order_is_descending(oracle):
    experts, hidden = 16, 32
    wr = np.zeros((experts, hidden), np.uint16)      # all logits 0 -> all scores 0.5
    bias = np.zeros(experts, np.float32)
    bias[[3, 9]] = 0.25                               # two equal leaders
    bias[12] = 0.5
    x = np.ones((1, hidden), np.float32)
    ids, wts, margin, scores = oracle.router(wr, bias, x, topk=4, routed_scale=2.0, mode=1)
    assert ids[0].tolist() == [12, 3, 9, 0]           # descending sel; ties by lowest index
    np.testing.assert_allclose(wts[0], np.full(4, 0.5 / 2.0 * 2.0), rtol=1e-6)
    assert margin[0] == 0.0                           # 4th and 5th are tied: flagged ambiguous
    assert np.allclose(scores, 0.5)


def test_expert_ffn_modes_and_numpy(oracle):
    rng = np.random.default_rng(2)
    hidden, inter = 256, 128
    _, gw = util.rand_i4(rng, inter, hidden)
    _, uw = util.rand_i4(rng, inter, hidden)
    _, dw = util.rand_i4(rng, hidden, inter)
    gs, us, ds = (util.rand_scales(rng, r, c // 32, 0.05) for r, c in ((inter, hidden), (inter, hidden), (hidden, inter)))
    x = oracle.bf16_round(rng.normal(size=hidden).astype(np.float32))
    wide = oracle.expert_ffn(gw, gs, uw, us, dw, ds, x, mode=0, round_out=False)
    exact = oracle.expert_ffn(gw, gs, uw, us, dw, ds, x, mode=1)
    G, U, D = (util.bf16_np_to_f32(oracle.i4_dequant(w, s)).astype(np.float64) for w, s in ((gw, gs), (uw, us), (dw, ds)))
    g, u = G @ x, U @ x
    ref = D @ (g / (1 + np.exp(-g)) * u)
    np.testing.assert_allclose(wide, ref, rtol=1e-4, atol=1e-6)
    util.assert_close(exact, ref, "ref_exact vs numpy")


def test_moe_layer_is_weighted_sum_plus_shared(oracle):
    rng = np.random.default_rng(3)
    hidden, inter, experts, topk, sh = 128, 64, 8, 2, 32
    wr = util.f32_to_bf16_np(rng.normal(0, 0.2, (experts, hidden)).astype(np.float32))
    bias = rng.normal(0, 0.01, experts).astype(np.float32)
    packs = {k: np.stack([util.rand_i4(rng, r, c)[1] for _ in range(experts)])
             for k, (r, c) in dict(g=(inter, hidden), u=(inter, hidden), d=(hidden, inter)).items()}
    scs = {k: np.stack([util.rand_scales(rng, r, c // 32, 0.05) for _ in range(experts)])
           for k, (r, c) in dict(g=(inter, hidden), u=(inter, hidden), d=(hidden, inter)).items()}
    sg, su = (util.f32_to_bf16_np(rng.normal(0, 0.1, (sh, hidden)).astype(np.float32)) for _ in range(2))
    sd = util.f32_to_bf16_np(rng.normal(0, 0.1, (hidden, sh)).astype(np.float32))
    x = oracle.bf16_round(rng.normal(size=(3, hidden)).astype(np.float32))
    slot_of = np.arange(experts, dtype=np.int32)
    out, ids, wts = oracle.moe_layer(wr, bias, slot_of, packs["g"], scs["g"], packs["u"], scs["u"], packs["d"], scs["d"],
                                     sg, su, sd, x, topk=topk, routed_scale=2.827, mode=0)
    for t in range(3):
        acc = np.zeros(hidden)
        for k in range(topk):
            e = int(ids[t, k])
            acc += wts[t, k] * oracle.expert_ffn(packs["g"][e], scs["g"][e], packs["u"][e], scs["u"][e], packs["d"][e],
                                                 scs["d"][e], x[t], mode=0, round_out=False).astype(np.float64)
        acc += oracle.bf16_mlp(sg, su, sd, x[t], mode=0, round_out=False)
        np.testing.assert_array_equal(out[t], oracle.bf16_round(acc.astype(np.float32)))
    # an absent expert is reported, not silently skipped
    slot_of[int(ids[0, 0])] = -1
    with pytest.raises(RuntimeError):
        oracle.moe_layer(wr, bias, slot_of, packs["g"], scs["g"], packs["u"], scs["u"], packs["d"], scs["d"], sg, su, sd,
                         x, topk=topk, mode=0)
    # ref_exact stays within the floating-point bar of the wide evaluation
    slot_of = np.arange(experts, dtype=np.int32)
    out1, ids1, _ = oracle.moe_layer(wr, bias, slot_of, packs["g"], scs["g"], packs["u"], scs["u"], packs["d"], scs["d"],
                                     sg, su, sd, x, topk=topk, mode=1)
    assert np.array_equal(ids, ids1)
    util.assert_close(out1, out, "moe ref_exact vs wide")


def test_rmsnorm(oracle):
    rng = np.random.default_rng(4)
    x = oracle.bf16_round(rng.normal(size=1536).astype(np.float32))
    w = util.f32_to_bf16_np(rng.normal(1, 0.1, 1536).astype(np.float32))
    a, b = oracle.rmsnorm(x, w, 1e-5, 0), oracle.rmsnorm(x, w, 1e-5, 1)
    ref = x / np.sqrt(np.mean(x.astype(np.float64) ** 2) + 1e-5) * util.bf16_np_to_f32(w)
    assert util.max_abs_rel(a, ref) < 5e-3 and util.max_abs_rel(b, ref) < 1e-2


def _tiny_mla(oracle, rng, seq):
    dims = dict(hidden=128, heads=4, qk_nope=32, qk_rope=16, v_head=32, q_rank=64, kv_rank=48)
    mk = lambda r, c, s=0.08: util.f32_to_bf16_np(rng.normal(0, s, (r, c)).astype(np.float32))
    W = dict(w_qa=mk(64, 128), qa_ln=util.f32_to_bf16_np(np.ones(64, np.float32)), w_qb=mk(4 * 48, 64),
             w_kva=mk(48 + 16, 128), kva_ln=util.f32_to_bf16_np(np.ones(48, np.float32)), w_kvb=mk(4 * 64, 48, 0.15))
    inv = oracle.yarn_inv_freq(16, 50000.0, 32.0, 32.0, 1.0, 4096.0)
    lat = np.zeros((seq, 64), np.float32)
    q = None
    for pos in range(seq):
        n = oracle.bf16_round(rng.normal(size=128).astype(np.float32))
        q, lat[pos] = oracle.mla_project(dims, W["w_qa"], W["qa_ln"], W["w_qb"], W["w_kva"], W["kva_ln"], n, pos, inv,
                                         1e-5, mode=1)
    return dims, W, q, lat


def test_mla_absorbed_equals_reference_form(oracle):
    rng = np.random.default_rng(5)
    dims, W, q, lat = _tiny_mla(oracle, rng, seq=70)   # spans two 64-token tiles of the reference's softmax
    ms = oracle.yarn_mscale(32.0, 1.0)
    ref_exact = oracle.mla_attend_ref(dims, W["w_kvb"], q, lat, ms, mode=1)
    ref_wide = oracle.mla_attend_ref(dims, W["w_kvb"], q, lat, ms, mode=0)
    absorbed = oracle.mla_attend_absorbed(dims, W["w_kvb"], q, util.f32_to_bf16_np(lat), ms)
    util.assert_close(ref_exact, ref_wide, "mla ref_exact vs wide")
    util.assert_close(absorbed, ref_wide, "absorbed vs non-absorbed")
    # the latent rows are bf16-exact, so the bf16 cache loses nothing
    assert np.array_equal(oracle.bf16_round(lat), lat)


def test_lm_head_argmax_lowest_id_wins(oracle):
    rng = np.random.default_rng(6)
    w = util.f32_to_bf16_np(rng.normal(0, 0.1, (50, 64)).astype(np.float32))
    w[40] = w[7]                                       # identical rows -> identical logits
    n = oracle.bf16_round(util.bf16_np_to_f32(w[7]) * 4)
    tok, best = oracle.lm_head_argmax(w, n, mode=1)
    assert tok == 7 and best > 0


def test_add_round(oracle):
    a = np.array([1.0, 0.00390625], np.float32)
    b = np.array([0.00390625, 0.00390625], np.float32)
    np.testing.assert_array_equal(oracle.add_round(a, b), np.array([1.0, 0.0078125], np.float32))
