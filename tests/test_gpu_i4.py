"""GPU parity, through the C ABI, of the INT4 kernels against the CPU oracle."""
import numpy as np
import pytest
import torch

import util

pytestmark = pytest.mark.gpu


def _dev_i4(rng, rows, cols, device, std=0.003):
    q, w = util.rand_i4(rng, rows, cols)
    s = util.rand_scales(rng, rows, cols // 32, std)
    return w, s, util.np_u32_to_torch(w, device), util.np_bf16_to_torch(s, device)


@pytest.mark.parametrize("rows,cols", [(1, 32), (7, 96), (16, 256), (2048, 7168), (7168, 2048), (0, 64)])
def test_dequant_bit_exact(cuda, oracle, rows, cols):
    from blok_b200 import lib
    rng = np.random.default_rng(rows + cols)
    w, s, dw, ds = _dev_i4(rng, rows, cols, cuda)
    if rows == 0:
        dw, ds = torch.zeros((0, cols // 8), dtype=torch.int32, device=cuda), torch.zeros((0, cols // 32), dtype=torch.bfloat16, device=cuda)
        assert lib.i4_dequant(dw, ds).shape == (0, cols)
        return
    got = util.t2np_bf16(lib.i4_dequant(dw, ds))
    assert np.array_equal(got, oracle.i4_dequant(w, s))


def test_dequant_all_nibbles_all_scales_bit_exact(cuda, oracle):
    """Every nibble value against a spread of bf16 scales, including subnormal and large ones."""
    from blok_b200 import lib
    scales = np.array([0x0001, 0x007F, 0x0080, 0x3A83, 0x3B44, 0x3F80, 0x4049, 0x7F00, 0x8001, 0xBB44], np.uint16)
    rows = len(scales)
    q = np.tile(np.arange(-8, 8, dtype=np.int8), (rows, 2))
    w = oracle.i4_pack(q)
    s = scales.reshape(rows, 1)
    got = util.t2np_bf16(lib.i4_dequant(util.np_u32_to_torch(w, cuda), util.np_bf16_to_torch(s, cuda)))
    assert np.array_equal(got, oracle.i4_dequant(w, s))


@pytest.mark.parametrize("rows,cols", [(16, 256), (64, 7168), (2048, 7168), (7168, 2048), (48, 512), (5, 96), (65, 2048)])
def test_i4_gemv_bf16(cuda, oracle, rows, cols):
    from blok_b200 import lib
    rng = np.random.default_rng(rows * 3 + cols)
    w, s, dw, ds = _dev_i4(rng, rows, cols, cuda)
    x = oracle.bf16_round(rng.normal(size=cols).astype(np.float32))
    y = util.t2np_f32(lib.i4_gemv(dw, ds, torch.from_numpy(x).to(cuda).bfloat16()))
    wide = oracle.i4_gemv(w, s, x, mode=0, round_out=True)
    util.assert_close(y, wide, "i4_gemv %dx%d" % (rows, cols))
    exact = oracle.i4_gemv(w, s, x, mode=1, round_out=True)
    util.assert_close(y, exact, "i4_gemv vs ref_exact")


def test_i4_gemv_f32_shim_matches_reference_rounding(cuda, oracle):
    """The fp32-signature shim keeps the reference's per-weight rounding; only the summation order differs."""
    from blok_b200 import lib
    rng = np.random.default_rng(9)
    rows, cols = 64, 7168
    w, s, dw, ds = _dev_i4(rng, rows, cols, cuda)
    x = oracle.bf16_round(rng.normal(size=cols).astype(np.float32))
    y = util.t2np_f32(lib.i4_gemv(dw, ds, torch.from_numpy(x).to(cuda)))
    exact = oracle.i4_gemv(w, s, x, mode=1, round_out=True)
    # both are bf16-rounded sums of identical products: they may differ by one bf16 ulp at most
    ulp = np.maximum(np.abs(exact), 1e-30) * 2.0 ** -7
    assert np.all(np.abs(y - exact) <= ulp)
    assert np.mean(y == exact) > 0.9


def test_i4_gemv_linearity(cuda, oracle):
    """Size-independent property at full size: W(ax) == a W(x) for a power of two."""
    from blok_b200 import lib
    rng = np.random.default_rng(10)
    w, s, dw, ds = _dev_i4(rng, 2048, 7168, cuda)
    x = torch.from_numpy(oracle.bf16_round(rng.normal(size=7168).astype(np.float32))).to(cuda).bfloat16()
    y1 = lib.i4_gemv(dw, ds, x).float()
    y4 = lib.i4_gemv(dw, ds, x * 4).float()
    assert torch.equal(y4, y1 * 4)
    y0 = lib.i4_gemv(dw, ds, torch.zeros_like(x)).float()
    assert torch.count_nonzero(y0) == 0


@pytest.mark.parametrize("hidden,inter,seed", [(256, 256, 1), (512, 768, 2), (7168, 2048, 0)])
def test_expert_ffn(cuda, oracle, hidden, inter, seed):
    """Config 0 at (7168, 2048, seed 0): one routed expert, batch 1."""
    from blok_b200 import lib
    rng = np.random.default_rng(seed)
    std = 0.003 if hidden == 7168 else 0.03
    gw, gs, dgw, dgs = _dev_i4(rng, inter, hidden, cuda, std)
    uw, us, duw, dus = _dev_i4(rng, inter, hidden, cuda, std)
    dw, ds, ddw, dds = _dev_i4(rng, hidden, inter, cuda, std)
    x = oracle.bf16_round(rng.normal(size=hidden).astype(np.float32))
    y = util.t2np_f32(lib.expert_ffn(dgw, dgs, duw, dus, ddw, dds, torch.from_numpy(x).to(cuda).bfloat16()))
    wide = oracle.expert_ffn(gw, gs, uw, us, dw, ds, x, mode=0, round_out=True)
    r, c = util.assert_close(y, wide, "expert_ffn")
    exact = oracle.expert_ffn(gw, gs, uw, us, dw, ds, x, mode=1)
    util.assert_close(y, exact, "expert_ffn vs ref_exact")
    print("expert_ffn %dx%d: max-abs-rel %.2e cosine %.7f" % (hidden, inter, r, c))


def test_expert_ffn_deterministic(cuda, oracle):
    from blok_b200 import lib
    rng = np.random.default_rng(3)
    args = []
    for r, c in ((2048, 7168), (2048, 7168), (7168, 2048)):
        _, _, a, b = _dev_i4(rng, r, c, cuda)
        args += [a, b]
    x = torch.randn(7168, device=cuda).bfloat16()
    y1 = lib.expert_ffn(*args, x)
    y2 = lib.expert_ffn(*args, x)
    assert torch.equal(y1, y2)


def test_bad_shapes_raise(cuda):
    from blok_b200 import lib
    w = torch.zeros((16, 8), dtype=torch.int32, device=cuda)
    s = torch.zeros((16, 2), dtype=torch.bfloat16, device=cuda)
    with pytest.raises(lib.BlokError):
        lib.i4_gemv(w, s, torch.zeros(32, dtype=torch.bfloat16, device=cuda))
    with pytest.raises(lib.BlokError):
        lib.i4_gemv(w.cpu(), s, torch.zeros(64, dtype=torch.bfloat16, device=cuda))
