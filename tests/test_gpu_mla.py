"""GPU parity of MLA decode attention (config 3) against the CPU oracle."""
import numpy as np
import pytest
import torch

import util

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def layer32(cuda):
    from blok_b200 import lib, synth
    w = synth.mla_weights(cuda, seed=3)
    return w, lib.MlaLayer(w, yarn_factor=32.0, max_batch=8, max_ctx=32768)


def _oracle_core(oracle, w_kvb, q_b, cache_b, seq, mscale):
    """q_b [64, 576] (absorbed | rope) -> o_lat [64, 512] in fp64: the latent-space attention itself."""
    scale = 1.0 / np.sqrt(192.0) * mscale * mscale
    K = util.bf16_np_to_f32(cache_b[:seq]).astype(np.float64)
    s = q_b.astype(np.float64) @ K.T * scale
    s -= s.max(axis=1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=1, keepdims=True)
    return p @ K[:, :512]


@pytest.mark.parametrize("B,seqs", [(1, [1]), (2, [31, 32]), (3, [33, 100, 257]), (8, [4097] * 8), (8, [5, 700, 64, 1, 4096, 333, 2048, 96])])
def test_attend_core(cuda, oracle, layer32, B, seqs):
    from blok_b200 import synth
    w, layer = layer32
    ctx = max(seqs) + 3
    cache = synth.latent_cache(B, ctx, cuda, seed=3)
    g = torch.Generator(device=cuda).manual_seed(5)
    q = (torch.randn((B, 64, 576), generator=g, device=cuda) * 0.3).bfloat16()
    seq = torch.tensor(seqs, dtype=torch.int32, device=cuda)
    o = layer.attend(q, cache, seq)
    torch.cuda.synchronize()
    o_h, q_h, c_h = util.t2np_f32(o), util.t2np_f32(q), util.t2np_bf16(cache)
    ms = oracle.yarn_mscale(32.0, 1.0)
    assert abs(layer.scale - ms * ms / np.sqrt(192.0)) < 1e-6
    for b in range(B):
        ref = _oracle_core(oracle, None, q_h[b], c_h[b], seqs[b], ms)
        util.assert_close(o_h[b], ref, "attend core b=%d seq=%d" % (b, seqs[b]))


def test_attend_long_context_one_sequence(cuda, oracle, layer32):
    """ctx 32768 (the long configuration) on one sequence, checked in full against fp64."""
    from blok_b200 import synth
    w, layer = layer32
    cache = synth.latent_cache(1, 32768, cuda, seed=4)
    g = torch.Generator(device=cuda).manual_seed(6)
    q = (torch.randn((1, 64, 576), generator=g, device=cuda) * 0.3).bfloat16()
    seq = torch.tensor([32768], dtype=torch.int32, device=cuda)
    o = util.t2np_f32(layer.attend(q, cache, seq))
    ref = _oracle_core(oracle, None, util.t2np_f32(q)[0], util.t2np_bf16(cache)[0], 32768, oracle.yarn_mscale(32.0, 1.0))
    util.assert_close(o[0], ref, "attend ctx 32768")


def test_attend_properties_at_full_size(cuda, layer32):
    """Size-independent checks at batch 8 x ctx 32768: splitting invariance and the convex-combination bound."""
    from blok_b200 import synth
    w, layer = layer32
    cache = synth.latent_cache(8, 32768, cuda, seed=5)
    g = torch.Generator(device=cuda).manual_seed(7)
    q = (torch.randn((8, 64, 576), generator=g, device=cuda) * 0.3).bfloat16()
    seq = torch.full((8,), 32768, dtype=torch.int32, device=cuda)
    o8 = layer.attend(q, cache, seq)
    # the same sequences one at a time use 148 splits instead of 18: the merged result must agree
    for b in (0, 7):
        o1 = layer.attend(q[b:b + 1].contiguous(), cache[b:b + 1].contiguous(), seq[b:b + 1].contiguous())
        # every probability enters the second product rounded to bf16 (src/kimi_exec.cu:466) relative to its split's own
        # reference maximum, so two splittings differ by that rounding: about 2^-9 of an output's typical size, a few
        # times that of the largest output at most
        assert util.max_abs_rel(util.t2np_f32(o1[0]), util.t2np_f32(o8[b])) < 1e-2
    # softmax weights are a convex combination: every output lies inside the range of the cached values
    lo = cache[:, :, :512].float().amin(dim=1, keepdim=True)
    hi = cache[:, :, :512].float().amax(dim=1, keepdim=True)
    assert torch.all(o8.float() >= lo - 1e-2) and torch.all(o8.float() <= hi + 1e-2)
    assert torch.equal(o8, layer.attend(q, cache, seq)), "deterministic"


@pytest.mark.parametrize("factor,B,ctxs", [(32.0, 2, [40, 7]), (64.0, 1, [130]), (32.0, 8, [4096] * 8),
                                           (32.0, 12, [90 + 3 * i for i in range(12)]),      # 9..64 entries: projections
                                           (32.0, 33, [20 + i for i in range(33)])])         # through the streaming kernel
def test_mla_decode_block(cuda, oracle, factor, B, ctxs):
    """The whole block: projections, norm, RoPE, cache append, attention, o_proj; factor 64 is the reference's own."""
    from blok_b200 import lib, synth
    w = synth.mla_weights(cuda, seed=3, std=0.02)
    layer = lib.MlaLayer(w, yarn_factor=factor, max_batch=max(8, B), max_ctx=8192)
    ctx_stride = max(ctxs) + 8
    cache = synth.latent_cache(B, ctx_stride, cuda, seed=9)
    before = cache.clone()
    n = synth.activations(B, 7168, cuda, 3)
    ctx_len = torch.tensor(ctxs, dtype=torch.int32, device=cuda)
    out = layer.decode(n, cache, ctx_len)
    torch.cuda.synchronize()
    wh = {k: util.t2np_bf16(v) for k, v in w.items()}
    inv = oracle.yarn_inv_freq(64, 50000.0, factor, 32.0, 1.0, 4096.0)
    ms = oracle.yarn_mscale(factor, 1.0)
    n_h, out_h = util.t2np_f32(n), util.t2np_f32(out)
    check = range(B) if B <= 2 else (0, B - 1)
    for b in check:
        pos = ctxs[b]
        qo, lat = oracle.mla_project(oracle.KIMI_MLA, wh["q_a"], wh["q_a_ln"], wh["q_b"], wh["kv_a"], wh["kv_a_ln"], n_h[b], pos,
                                     inv, 1e-5, mode=1)
        got_row = util.t2np_f32(cache[b, pos])
        # the appended row: same arithmetic as the reference up to summation order and the last place of cosf/sinf
        assert np.mean(np.abs(got_row - lat) <= 2.0 ** -6 * np.maximum(np.abs(lat), 0.05)) > 0.98
        util.assert_close(got_row, lat, "latent row")
        rows = np.concatenate([util.t2np_bf16(before[b, :pos]), util.f32_to_bf16_np(lat)[None]], axis=0)
        av = oracle.mla_attend_absorbed(oracle.KIMI_MLA, wh["kv_b"], qo, rows, ms)
        ref = oracle.bf16_gemv(wh["o"], av, mode=0, round_out=True)
        util.assert_close(out_h[b], ref, "mla block b=%d" % b)
    # rows other than the appended one are untouched
    mask = torch.ones_like(cache, dtype=torch.bool)
    for b in range(B):
        mask[b, ctxs[b]] = False
    assert torch.equal(cache[mask], before[mask])
    layer.close()


def test_mla_rejects_bad_arguments(cuda, layer32):
    from blok_b200 import lib
    w, layer = layer32
    q = torch.zeros((9, 64, 576), dtype=torch.bfloat16, device=cuda)
    with pytest.raises(lib.BlokError):
        layer.attend(q, torch.zeros((9, 4, 576), dtype=torch.bfloat16, device=cuda), torch.ones(9, dtype=torch.int32, device=cuda))


def test_position_outside_the_cache_is_reported_not_stored(cuda, layer32):
    """ctx_len lives on the device, so a sequence already at its capacity cannot be refused before the launch: the
    kernel must skip the store (the row would land in the NEXT sequence's first row), keep its attention inside the
    sequence's rows, and blok_mla_layer_check must report the entry.  (The reference dies on the host, :205.)"""
    from blok_b200 import lib, synth
    w, layer = layer32
    ctx = 64
    cache = synth.latent_cache(3, ctx, cuda, seed=9)
    before = cache.clone()
    n = synth.activations(3, 7168, cuda, 9)
    ctx_len = torch.tensor([10, ctx, 20], dtype=torch.int32, device=cuda)     # entry 1 is full: position 64 of 64 rows
    out = layer.decode(n, cache, ctx_len)
    with pytest.raises(lib.BlokError) as e:
        layer.check()
    assert e.value.code == -2 and "entry 1" in str(e.value)
    layer.check()                                                            # reported once, then clear
    changed = (cache != before).any(dim=2)
    assert changed[0, 10] and changed[2, 20] and int(changed.sum()) == 2     # only the two legal rows were written
    assert torch.isfinite(out.float()).all()
    # a legal call afterwards is unaffected
    ctx_len2 = torch.tensor([11, 5, 21], dtype=torch.int32, device=cuda)
    layer.decode(n, cache, ctx_len2)
    layer.check()
