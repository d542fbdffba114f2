"""The entry point for callers that cannot allocate device memory: blok_expert_ffn_static keeps its intermediate
vector in an array built into the library instead of a caller workspace.  Checked through the C ABI against
blok_expert_ffn on the same inputs, on two calls in a row (the array keeps the first call's contents when the
second one starts).  Collected last so that a failure here cannot hide the other tests."""
import ctypes as C

import numpy as np
import pytest
import torch

import util

pytestmark = pytest.mark.gpu


def _expert(rng, hidden, inter, device):
    out = []
    for rows, cols in ((inter, hidden), (inter, hidden), (hidden, inter)):
        _, w = util.rand_i4(rng, rows, cols)
        s = util.rand_scales(rng, rows, cols // 32, 0.003 if hidden >= 4096 else 0.03)
        out += [util.np_u32_to_torch(w, device), util.np_bf16_to_torch(s, device)]
    return out


@pytest.mark.parametrize("hidden,inter", [(7168, 2048), (512, 768)])
def test_static_scratch_matches_workspace_entry_point(cuda, hidden, inter):
    from blok_b200 import lib
    rng = np.random.default_rng(hidden + inter)
    first, second = _expert(rng, hidden, inter, cuda), _expert(rng, hidden, inter, cuda)
    xs = torch.from_numpy(rng.normal(size=(2, hidden)).astype(np.float32)).to(cuda).bfloat16()
    y = torch.empty(hidden, dtype=torch.bfloat16, device=cuda)
    for call, (weights, x) in enumerate(((first, xs[0]), (second, xs[1]))):
        expect = lib.expert_ffn(*weights, x.contiguous())
        before = torch.cuda.memory_allocated()
        got = lib.expert_ffn_static(*weights, x.contiguous(), out=y)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before, "the call must not allocate through torch either"
        util.assert_close(util.t2np_f32(got), util.t2np_f32(expect), "static scratch, call %d" % call)
        assert torch.equal(got, expect), "same kernels, same inputs: the bits must agree (call %d)" % call


def test_static_scratch_rejects_sizes_beyond_its_array(cuda):
    from blok_b200 import lib
    l = lib.load()
    limit = l.blok_expert_ffn_static_max_inter()
    assert limit >= 2048
    p = C.c_void_p(256)  # validation fails before any launch
    rc = l.blok_expert_ffn_static(p, p, p, p, p, p, p, p, 7168, limit + 256, None)
    assert rc == -6
    assert b"exceeds the built-in scratch" in l.blok_last_error()
