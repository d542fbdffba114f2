"""The integer tensor-core consumer of the INT4 mat-vec (BLOK_I4_GEMV_IMPL=imma, csrc/i4_imma.cuh) on the GPU.

Same contract as matvec_i4_bf16_scale_k (src/kimi_exec.cu:300-323) within the floating-point bar.  What it rounds
differs from the reference: the activations of a 32-column scale group become 15-bit block integers
(X = round(x * 2^(13 - E)), E the group's largest exponent), the integer sums are exact, and the weight scale is
applied to the group sum; the reference rounds every dequantised weight to bf16 (:312).  The bounds below follow
from that: per group at most half an integer unit per column."""
import numpy as np
import pytest
import torch

import util

pytestmark = pytest.mark.gpu


def _group_exponent(x):
    """floor(log2) of the largest magnitude of every 32-column group (0 for an all-zero group)."""
    m = np.abs(x.reshape(-1, 32)).max(axis=1)
    return np.where(m > 0, np.floor(np.log2(np.maximum(m, 1e-300))), 0.0)


@pytest.mark.parametrize("rows,cols", [(16, 128), (64, 7168), (2048, 7168), (7168, 2048), (48, 384)])
def test_i4_gemv_integer_path(cuda, oracle, monkeypatch, rows, cols):
    from blok_b200 import lib
    from test_gpu_i4 import _dev_i4
    rng = np.random.default_rng(rows * 5 + cols)
    w, s, dw, ds = _dev_i4(rng, rows, cols, cuda)
    x = oracle.bf16_round(rng.normal(size=cols).astype(np.float32))
    xd = torch.from_numpy(x).to(cuda).bfloat16()
    base = util.t2np_f32(lib.i4_gemv(dw, ds, xd))
    monkeypatch.setenv("BLOK_I4_GEMV_IMPL", "imma")
    y = util.t2np_f32(lib.i4_gemv(dw, ds, xd))
    monkeypatch.delenv("BLOK_I4_GEMV_IMPL")
    wide = oracle.i4_gemv(w, s, x, mode=0, round_out=True)
    util.assert_close(y, wide, "integer-path i4_gemv %dx%d" % (rows, cols))
    util.assert_close(y, base, "integer path vs the default path")

    # the stated error model, against the sum with NO rounding of the dequantised weights (fp64):
    #   |y - sum_c q s x| <= sum_groups s_g * 2^(E_g - 14) * sum_c |q_c|   (half a unit of X per column)
    #                        + fp32 accumulation over the groups + the final bf16 rounding
    q = ((w[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))) & 0xF).astype(np.int64).reshape(rows, cols) - 8
    sf = util.bf16_np_to_f32(s).astype(np.float64)
    plain = (q.reshape(rows, cols // 32, 32) * x.astype(np.float64).reshape(1, cols // 32, 32)).sum(-1)
    exact = (plain * sf).sum(-1)
    unit = np.exp2(_group_exponent(x.astype(np.float64)) - 14.0)
    quant = (np.abs(q).reshape(rows, cols // 32, 32).sum(-1) * sf * unit[None, :]).sum(-1)
    mag = (np.abs(plain) * sf).sum(-1)
    bound = quant + mag * 2.0 ** -20 + np.abs(exact) * 2.0 ** -8 + 1e-30
    assert np.all(np.abs(y - exact) <= bound), float(np.max(np.abs(y - exact) / bound))
    # that is far inside the bar: what is left is the bf16 rounding of the result itself (2^-9 relative)
    assert util.max_abs_rel(y, exact) < 2.0 ** -8

    if cols % 256 == 0:
        # here the default is the bf16-operand tensor-core path, which does not round q * scale either: both are bf16
        # roundings of nearly the same sum, a step of the last place apart at most and equal almost everywhere.
        # (Below 256 columns the default is the scalar kernel, which keeps the reference's per-weight rounding.)
        near = np.abs(y - base) <= np.maximum(np.abs(base) * 2.0 ** -7, mag * 2.0 ** -12)
        assert np.all(near)
        assert np.mean(y == base) > 0.8
    # zero in, zero out; scaling the input by a power of two scales the output exactly
    monkeypatch.setenv("BLOK_I4_GEMV_IMPL", "imma")
    assert torch.count_nonzero(lib.i4_gemv(dw, ds, torch.zeros_like(xd))) == 0
    assert torch.equal(lib.i4_gemv(dw, ds, xd * 8).float(), lib.i4_gemv(dw, ds, xd).float() * 8)
