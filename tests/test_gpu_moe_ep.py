"""The expert-parallel layer under the C ABI (blok_moe_ep_*) on ONE GPU: with a world of one rank the whole exchange
(count table, plan, dispatch into the receive buffer, grouped GEMM, combine from the result buffer) runs against the
rank's own buffers, and the result must equal blok_moe_batched bit for bit: the same kernels compute every row and the
combine adds the slots in the same order.  (Two ranks: tests/test_gpu_ep.py.)"""
import pytest
import torch

import util

pytestmark = pytest.mark.gpu


def _small_layer(cuda, seed, shared=512):
    from blok_b200 import synth
    w = synth.moe_layer_weights(cuda, seed=seed, hidden=1024, inter=512, experts=128, shared_inter=shared)
    for k in ("gate_s", "up_s", "down_s"):
        w[k] = (w[k].float() * 8).bfloat16()
    w["router_w"] = (w["router_w"].float() * 20).bfloat16()
    return w


@pytest.mark.parametrize("impl", ["mma", "tc"])
def test_one_rank_world_equals_the_batched_layer(cuda, monkeypatch, impl):
    from blok_b200 import lib, synth
    monkeypatch.setenv("BLOK_WGEMM_IMPL", impl)
    w = _small_layer(cuda, 51)
    comm = lib.Comm(rank=0, world=1)
    ep = lib.MoeEp(comm, w, max_tokens=300)
    full = lib.MoeLayer(w, max_tokens=300)
    for T in (1, 20, 300, 7):                       # several passes on one handle: the flags carry the pass number
        x = synth.activations(T, 1024, cuda, 60 + T)
        y, ids, wts = ep.forward(x, return_routing=True)
        ep.check()
        ref, rid, rw = full.batched(x, return_routing=True)
        assert torch.equal(ids, rid) and torch.equal(wts, rw)
        assert torch.equal(y, ref), "T=%d: max diff %g" % (T, float((y.float() - ref.float()).abs().max()))
        st = ep.stats()
        assert st["assignments"] == T * 8 and st["remote"] == 0 and st["received"] == T * 8
    # a pass without tokens is legal (a rank whose share of the batch is empty still takes part)
    assert ep.forward(x[:0].contiguous()).shape == (0, 1024)
    ep.check()
    assert ep.stats()["received"] == 0
    with pytest.raises(lib.BlokError):
        ep.forward(synth.activations(301, 1024, cuda, 1))
    ep.close(); full.close(); comm.close()


def test_one_rank_world_without_shared_expert_and_full_size_rows(cuda):
    """hidden 7168 rows (the row size the exchange moves in config 2), no shared expert."""
    from blok_b200 import lib, synth
    w = synth.moe_layer_weights(cuda, seed=52, hidden=7168, inter=512, experts=128, shared_inter=0)
    comm = lib.Comm(rank=0, world=1)
    ep = lib.MoeEp(comm, w, max_tokens=64)
    full = lib.MoeLayer(w, max_tokens=64)
    x = synth.activations(33, 7168, cuda, 5)
    y = ep.forward(x)
    ep.check()
    assert torch.equal(y, full.batched(x))
    ep.close(); full.close(); comm.close()


def test_shard_must_match_the_rank(cuda):
    from blok_b200 import lib
    w = _small_layer(cuda, 53)
    comm = lib.Comm(rank=0, world=1)
    half = dict(w)
    for k in ("gate_w", "gate_s", "up_w", "up_s", "down_w", "down_s"):
        half[k] = w[k][:64].contiguous()
    with pytest.raises(lib.BlokError) as e:
        lib.MoeEp(comm, half, max_tokens=8)      # 64 of 128 experts on a world of one rank
    assert e.value.code == -2
    comm.close()
