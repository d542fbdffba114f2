"""The CPU oracle against known-answer vectors of the upstream packages the
reference pins its semantics to (tests/golden/third_party.npz, made by
tests/golden/make_third_party_golden.py)."""
import os

import numpy as np
import pytest

import util

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "third_party.npz"))


def test_pack_layout_matches_compressed_tensors(oracle):
    q, words = G["pack_q"], G["pack_words"]
    assert np.array_equal(oracle.i4_pack(q), words)
    # documented pattern: q = -8..7 packs to 0x76543210, 0xfedcba98
    assert words[0, 0] == 0x76543210 and words[0, 1] == 0xFEDCBA98
    # decode rule of the reference (src/kimi_exec.cu:311) recovers q: scale 1.0 dequant == q
    ones = np.full((q.shape[0], q.shape[1] // 32), 0x3F80, np.uint16)
    deq = util.bf16_np_to_f32(oracle.i4_dequant(words, ones))
    assert np.array_equal(deq, q.astype(np.float32))


def test_numpy_packer_agrees(oracle):
    rng = np.random.default_rng(0)
    q, w = util.rand_i4(rng, 8, 64)
    assert np.array_equal(oracle.i4_pack(q), w)


@pytest.mark.parametrize("mode", [0, 1])
def test_router_matches_hf_deepseek_v3(oracle, mode):
    wr = util.f32_to_bf16_np(G["router_w"])          # the weights were made bf16-exact
    assert np.array_equal(util.bf16_np_to_f32(wr), G["router_w"])
    ids, wts, margin, _ = oracle.router(wr, G["router_bias"], G["router_x"], topk=8, routed_scale=2.827, mode=mode)
    for t in range(ids.shape[0]):
        assert set(ids[t].tolist()) == set(G["router_idx"][t].tolist()), "token %d" % t
        got = dict(zip(ids[t].tolist(), wts[t].tolist()))
        for e, w in zip(G["router_idx"][t].tolist(), G["router_wts"][t].tolist()):
            assert abs(got[e] - w) <= 2e-6 * max(1.0, abs(w))
    assert np.all(margin > 0)


@pytest.mark.parametrize("factor", [32, 64])
def test_yarn_matches_hf(oracle, factor):
    f = oracle.yarn_inv_freq(64, 50000.0, float(factor), 32.0, 1.0, 4096.0)
    np.testing.assert_allclose(f, G["yarn_inv_freq_%d" % factor], rtol=2e-6)
    ms = oracle.yarn_mscale(float(factor), 1.0)
    assert abs(ms - float(G["yarn_mscale_%d" % factor])) < 1e-6
    # mscale == mscale_all_dim makes HF's cos/sin post-scale 1, as in the reference (no mscale in rope_k)
    assert abs(float(G["yarn_attn_factor_%d" % factor]) - 1.0) < 1e-6


def test_yarn_constants():
    import math
    # values derived from the reference's constants (src/kimi_exec.cu:183-185, :428-429)
    assert abs((0.1 * math.log(64.0) + 1.0) - 1.41589) < 1e-5
    assert abs((0.1 * math.log(32.0) + 1.0) - 1.34657) < 1e-5


def test_rope_matches_hf_up_to_bf16_rounding(oracle):
    # the oracle keeps the reference's bf16 rounding of cos, sin and products (:351-356);
    # HF evaluates in fp32, so agreement is to bf16 precision on a bf16-exact input.
    x = util.bf16_np_to_f32(util.f32_to_bf16_np(G["rope_x"]))
    cs = oracle.rope_table(G["yarn_inv_freq_32"], int(G["rope_pos"]))
    y = oracle.rope_vec(x, cs)
    ang = int(G["rope_pos"]) * G["yarn_inv_freq_32"].astype(np.float64)
    x0, x1 = x[0::2].astype(np.float64), x[1::2].astype(np.float64)
    exact = np.concatenate([x0 * np.cos(ang) - x1 * np.sin(ang), x1 * np.cos(ang) + x0 * np.sin(ang)])
    assert np.max(np.abs(y - exact)) < 3e-2
    # and HF's own output on the unrounded input equals the same closed form
    x0, x1 = G["rope_x"][0::2].astype(np.float64), G["rope_x"][1::2].astype(np.float64)
    hf = np.concatenate([x0 * np.cos(ang) - x1 * np.sin(ang), x1 * np.cos(ang) + x0 * np.sin(ang)])
    np.testing.assert_allclose(G["rope_y"], hf, atol=2e-5)
