"""Pins the CPU oracle to the reference's own kernels.

oracle/_ref/libblok_ref.so is the reference executor's translation unit compiled
from its source (oracle/build.py) with launchers for its kernels
(oracle/ref_shim/ref_shim.cu).  These tests run those kernels on the GPU and
compare them with the oracle's ORC_REF_EXACT mode, which restates the same
arithmetic, schedule included.  They skip when the prebuilt library is absent.
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import util

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref", "libblok_ref.so")


@pytest.fixture(scope="module")
def ref(cuda):
    if not os.path.exists(REF):
        pytest.skip("oracle/_ref/libblok_ref.so not built (reference checkout absent at build time)")
    return C.CDLL(REF)


def P(t):
    return C.c_void_p(t.data_ptr())


def test_ref_i4_matvec(ref, cuda, oracle):
    rng = np.random.default_rng(0)
    for rows, cols in ((64, 7168), (128, 2048)):
        _, w = util.rand_i4(rng, rows, cols)
        s = util.rand_scales(rng, rows, cols // 32)
        x = oracle.bf16_round(rng.normal(size=cols).astype(np.float32))
        dw, ds = util.np_u32_to_torch(w, cuda), util.np_bf16_to_torch(s, cuda)
        dx, dy = torch.from_numpy(x).to(cuda), torch.zeros(rows, device=cuda)
        assert ref.ref_matvec_i4(P(dw), P(ds), P(dx), P(dy), rows, cols) == 0
        got = dy.cpu().numpy()
        exact = oracle.i4_gemv(w, s, x, mode=1, round_out=True)
        # same products, same schedule, fused multiply-add on both sides: identical bits
        assert np.array_equal(got, exact), "mismatch in %d of %d rows" % (np.sum(got != exact), rows)


def test_ref_bf16_matvec_and_logits(ref, cuda, oracle):
    rng = np.random.default_rng(1)
    rows, cols = 64, 7168
    w = util.f32_to_bf16_np(rng.normal(0, 0.006, (rows, cols)).astype(np.float32))
    x = oracle.bf16_round(rng.normal(size=cols).astype(np.float32))
    dw, dx, dy = util.np_bf16_to_torch(w, cuda), torch.from_numpy(x).to(cuda), torch.zeros(rows, device=cuda)
    assert ref.ref_matvec_bf16(P(dw), P(dx), P(dy), rows, cols) == 0
    assert np.array_equal(dy.cpu().numpy(), oracle.bf16_gemv(w, x, mode=1, round_out=True))
    assert ref.ref_matvec_bf16_f32(P(dw), P(dx), P(dy), rows, cols) == 0
    assert np.array_equal(dy.cpu().numpy(), oracle.bf16_gemv(w, x, mode=1, round_out=False))


def test_ref_silu_rmsnorm_add(ref, cuda, oracle):
    rng = np.random.default_rng(2)
    a = oracle.bf16_round(rng.normal(0, 2, 2048).astype(np.float32))
    b = oracle.bf16_round(rng.normal(0, 2, 2048).astype(np.float32))
    da, db, dy = torch.from_numpy(a).to(cuda), torch.from_numpy(b).to(cuda), torch.zeros(2048, device=cuda)
    assert ref.ref_silu_mul(P(da), P(db), P(dy), 2048) == 0
    got, exp = dy.cpu().numpy(), oracle.silu_mul(a, b, mode=1)
    # expf differs by an ulp between the device and libm; after two bf16 roundings almost all agree
    assert np.mean(got == exp) > 0.995 and util.max_abs_rel(got, exp) < 8e-3
    x = oracle.bf16_round(rng.normal(0, 3, 7168).astype(np.float32))
    w = util.f32_to_bf16_np(rng.normal(1, 0.1, 7168).astype(np.float32))
    dx, dw, dy = torch.from_numpy(x).to(cuda), util.np_bf16_to_torch(w, cuda), torch.zeros(7168, device=cuda)
    assert ref.ref_rmsnorm(P(dx), P(dw), P(dy), 7168) == 0
    got, exp = dy.cpu().numpy(), oracle.rmsnorm(x, w, 1e-5, mode=1)
    assert np.mean(got == exp) > 0.98 and util.max_abs_rel(got, exp) < 8e-3
    da = torch.from_numpy(a).to(cuda)
    assert ref.ref_add(P(da), P(db), 2048) == 0
    assert np.array_equal(da.cpu().numpy(), oracle.add_round(a, b))


def test_ref_router_tail(ref, cuda, oracle):
    rng = np.random.default_rng(3)
    experts, hidden = 384, 7168
    wr = util.f32_to_bf16_np(rng.normal(0, 0.006, (experts, hidden)).astype(np.float32))
    bias16 = util.f32_to_bf16_np(rng.normal(0, 0.01, experts).astype(np.float32))
    for trial in range(4):
        x = oracle.bf16_round(rng.normal(size=hidden).astype(np.float32))
        dw, dx = util.np_bf16_to_torch(wr, cuda), torch.from_numpy(x).to(cuda)
        logits, select = torch.zeros(experts, device=cuda), torch.zeros(experts, device=cuda)
        assert ref.ref_matvec_bf16_f32(P(dw), P(dx), P(logits), experts, hidden) == 0
        ids = torch.zeros(8, dtype=torch.int16, device=cuda)
        wts = torch.zeros(8, device=cuda)
        assert ref.ref_router_tail(P(logits), P(select), P(util.np_bf16_to_torch(bias16, cuda)), P(ids), P(wts)) == 0
        oid, owt, margin, _ = oracle.router(wr, util.bf16_np_to_f32(bias16), x[None], topk=8, routed_scale=2.827, mode=1)
        if margin[0] > 1e-6:
            assert util.ids_np(ids).tolist() == oid[0].tolist()
            np.testing.assert_allclose(wts.cpu().numpy(), owt[0], rtol=1e-5)


def test_ref_rope(ref, cuda, oracle):
    rng = np.random.default_rng(4)
    q = oracle.bf16_round(rng.normal(size=64 * 192).astype(np.float32))
    k = oracle.bf16_round(rng.normal(size=64 * 192).astype(np.float32))
    inv = oracle.yarn_inv_freq(64, 50000.0, 64.0, 32.0, 1.0, 4096.0)   # the reference hard-codes factor 64
    for pos in (0, 1, 777, 40000):
        dq, dk = torch.from_numpy(q).to(cuda), torch.from_numpy(k).to(cuda)
        qr, kr = torch.zeros_like(dq), torch.zeros_like(dk)
        assert ref.ref_rope(P(dq), P(dk), P(qr), P(kr), pos) == 0
        cs = oracle.rope_table(inv, pos)
        got = qr.cpu().numpy().reshape(64, 192)
        exp = np.stack([np.concatenate([q.reshape(64, 192)[h, :128], oracle.rope_vec(q.reshape(64, 192)[h, 128:], cs)])
                        for h in range(64)])
        assert np.array_equal(got[:, :128], exp[:, :128])
        # powf/cosf/sinf differ in the last place between device and libm; large angles amplify it
        tol = 2e-2 if pos < 1000 else 1.5e-1
        assert np.mean(np.abs(got[:, 128:] - exp[:, 128:]) <= tol * np.maximum(1.0, np.abs(exp[:, 128:]))) > 0.97


def test_ref_tiled_attention(ref, cuda, oracle):
    """The reference's three-pass softmax over materialised K/V against the oracle's restatement of it, and the
    absorbed latent-cache form against both."""
    rng = np.random.default_rng(5)
    dims = oracle.KIMI_MLA
    seq = 150
    w_kvb = util.f32_to_bf16_np(rng.normal(0, 0.03, (64 * 256, 512)).astype(np.float32))
    lat = oracle.bf16_round(rng.normal(size=(seq, 576)).astype(np.float32))
    q = oracle.bf16_round(rng.normal(0, 0.3, (64, 192)).astype(np.float32))
    # materialise K and V with the reference's own kernels (kv_b mat-vec, split, k_pe fill)
    K = torch.zeros((seq, 64 * 192), device=cuda)
    V = torch.zeros((seq, 64 * 128), device=cuda)
    dwk = util.np_bf16_to_torch(w_kvb, cuda)
    kv = torch.zeros(64 * 256, device=cuda)
    for t in range(seq):
        dl = torch.from_numpy(lat[t]).to(cuda)
        assert ref.ref_matvec_bf16(P(dwk), P(dl), P(kv), 64 * 256, 512) == 0
        assert ref.ref_split_kv(P(kv), P(K[t]), P(V[t]), C.c_void_p(dl.data_ptr() + 512 * 4)) == 0
    out = torch.zeros(64 * 128, device=cuda)
    score, hmax, hsum = torch.zeros(64 * 64, device=cuda), torch.zeros(64, device=cuda), torch.zeros(64, device=cuda)
    dq = torch.from_numpy(q).to(cuda)
    assert ref.ref_tiled_attention(P(K), P(V), seq, 64, P(dq), P(out), P(score), P(hmax), P(hsum)) == 0
    got = out.cpu().numpy()
    ms = oracle.yarn_mscale(64.0, 1.0)
    exact = oracle.mla_attend_ref(dims, w_kvb, q, lat, ms, mode=1)
    assert util.max_abs_rel(got, exact) < 1e-2 and util.cosine(got, exact) > 0.99995
    absorbed = oracle.mla_attend_absorbed(dims, w_kvb, q, util.f32_to_bf16_np(lat), ms)
    util.assert_close(absorbed, got, "absorbed oracle vs reference kernels")
