"""GPU parity of the batched routed-MoE layer (config 2) against the oracle and against the batch-1 path."""
import numpy as np
import pytest
import torch

import util
from test_gpu_moe_decode import _host_layer

pytestmark = pytest.mark.gpu
MARGIN = 2e-6


def _oracle_layer(oracle, w, x, ids_needed, topk=8):
    slot_of, packs, scs, shared = _host_layer(w, ids_needed)
    return oracle.moe_layer(util.t2np_bf16(w["router_w"]), util.t2np_f32(w["router_bias"]), slot_of, packs["gate_w"],
                            scs["gate_s"], packs["up_w"], scs["up_s"], packs["down_w"], scs["down_s"], shared[0], shared[1],
                            shared[2], util.t2np_f32(x), topk=topk, mode=0)


# the mma.sync kernel and the tcgen05 kernels, whatever the size; "auto": the library's own choice, which sends groups of
# up to four tokens through the mat-vec-style kernel (wgemv_small.cu) and the rest through the kernel the size picks
@pytest.mark.parametrize("impl", ["mma", "tc", "auto"])
@pytest.mark.parametrize("T,hidden,inter,experts,shared,seed", [(40, 1024, 512, 128, 512, 31), (1, 1024, 512, 128, 512, 32),
                                                                (64, 7168, 2048, 384, 2048, 2), (130, 512, 512, 128, 0, 33),
                                                                (7, 1024, 512, 128, 512, 34)])
def test_moe_batched_vs_oracle(cuda, oracle, monkeypatch, impl, T, hidden, inter, experts, shared, seed):
    from blok_b200 import lib, synth
    if impl == "auto":
        monkeypatch.delenv("BLOK_WGEMM_IMPL", raising=False)
    else:
        monkeypatch.setenv("BLOK_WGEMM_IMPL", impl)
    w = synth.moe_layer_weights(cuda, seed=seed, hidden=hidden, inter=inter, experts=experts, shared_inter=shared)
    if hidden < 7168:
        for k in ("gate_s", "up_s", "down_s"):
            w[k] = (w[k].float() * 8).bfloat16()
        w["router_w"] = (w["router_w"].float() * 20).bfloat16()
    layer = lib.MoeLayer(w, max_tokens=max(T, 2))
    x = synth.activations(T, hidden, cuda, seed)
    y, ids, wts = layer.batched(x, return_routing=True)
    layer.check()  # no tensor-core tile gave up on a barrier
    ids_h = util.ids_np(ids)
    oid, owt, margin, _ = oracle.router(util.t2np_bf16(w["router_w"]), util.t2np_f32(w["router_bias"]), util.t2np_f32(x), mode=0)
    clear = margin > MARGIN
    assert clear.mean() > 0.95
    for t in np.nonzero(clear)[0]:
        assert set(ids_h[t].tolist()) == set(oid[t].tolist()), "token %d" % t
    out, _, _ = _oracle_layer(oracle, w, x, list(ids_h.ravel()) + list(oid.ravel()))
    yh = util.t2np_f32(y)
    same = np.all(ids_h == oid, axis=1)
    for t in np.nonzero(same)[0]:
        util.assert_close(yh[t], out[t], "batched token %d" % t)
    assert same.mean() > 0.9
    assert torch.equal(y, layer.batched(x)), "deterministic"
    layer.close()


def test_moe_batched_agrees_with_decode_path_at_2048_tokens(cuda):
    """T = 2048 (config 2's large case): every token of the batch must match the batch-1 kernel on the same token."""
    from blok_b200 import lib, synth
    w = synth.moe_layer_weights(cuda, seed=2)
    layer = lib.MoeLayer(w, max_tokens=2048)
    x = synth.activations(2048, 7168, cuda, 2)
    y, ids, wts = layer.batched(x, return_routing=True)
    counts = torch.bincount(ids.view(torch.int16).long().ravel() & 0xFFFF, minlength=384)
    assert int(counts.sum()) == 2048 * 8 and int((counts > 0).sum()) > 350
    for t in (0, 1, 777, 2047):
        y1, i1, w1 = layer.decode(x[t].contiguous(), return_routing=True)
        if torch.equal(i1, ids[t]):
            assert util.max_abs_rel(util.t2np_f32(y[t]), util.t2np_f32(y1)) < 1e-2
            assert util.cosine(util.t2np_f32(y[t]), util.t2np_f32(y1)) > 0.9999
    np.testing.assert_allclose(util.t2np_f32(wts).sum(axis=1), 2.827, rtol=1e-5)
    layer.close()


def test_moe_batched_2048_tokens_against_the_oracle(cuda, oracle):
    """Config 2's large case at full size (T = 2048, 384 experts): the routing of EVERY token against the oracle, in
    selection order, and the layer output of 64 tokens spread over the batch against the oracle's layer."""
    from blok_b200 import lib, synth
    w = synth.moe_layer_weights(cuda, seed=2)
    layer = lib.MoeLayer(w, max_tokens=2048)
    x = synth.activations(2048, 7168, cuda, 2)
    y, ids, wts = layer.batched(x, return_routing=True)
    layer.check()
    ids_h, wts_h = util.ids_np(ids), util.t2np_f32(wts)
    oid, owt, margin, _ = oracle.router(util.t2np_bf16(w["router_w"]), util.t2np_f32(w["router_bias"]), util.t2np_f32(x), mode=0)
    # a token's selection is beyond doubt when the 8th and 9th candidates are apart (margin) and so are the selected ones
    # among themselves (their weights are the scores, normalised: distinct weights, distinct scores)
    gaps = np.abs(np.diff(np.sort(owt, axis=1), axis=1)).min(axis=1)
    clear = (margin > MARGIN) & (gaps > 1e-6)
    assert clear.mean() > 0.9
    assert np.array_equal(ids_h[clear], oid[clear]), "top-k ids, in selection order"
    np.testing.assert_allclose(wts_h[clear], owt[clear], rtol=2e-5)
    sample = np.nonzero(clear)[0][:: max(1, int(clear.sum()) // 64)][:64]
    assert len(sample) == 64
    xs = x[torch.from_numpy(sample).to(cuda)]
    out, _, _ = _oracle_layer(oracle, w, xs, list(oid[sample].ravel()))
    yh = util.t2np_f32(y)
    worst = 0.0
    for i, t in enumerate(sample):
        r, c = util.assert_close(yh[t], out[i], "T=2048 token %d" % t)
        worst = max(worst, r)
    print("T=2048: %d tokens routed as the oracle routes them, 64 outputs checked, worst max-abs-rel %.2e" % (int(clear.sum()), worst))
    layer.close()


@pytest.mark.parametrize("impl", ["mma", "tc", "auto"])
def test_experts_grouped_handles_empty_and_ragged_groups(cuda, oracle, monkeypatch, impl):
    """Assignments concentrated on few experts (others get zero tokens), more than one 64-token tile for one expert.
    Left to itself ("auto") the library sends all of them through the small-group kernel: the larger groups are few, so
    it takes the 64-token tile (sixteen passes of four tokens) and the group of nine as well."""
    from blok_b200 import lib, synth
    monkeypatch.setenv("BLOK_WGEMM_IMPL", impl)
    hidden, inter, experts = 512, 512, 128
    w = synth.moe_layer_weights(cuda, seed=41, hidden=hidden, inter=inter, experts=experts, shared_inter=0)
    for k in ("gate_s", "up_s", "down_s"):
        w[k] = (w[k].float() * 8).bfloat16()
    layer = lib.MoeLayer(w, max_tokens=64)
    x = synth.activations(30, hidden, cuda, 41)
    e = torch.tensor([5] * 70 + [127] * 3 + [0] + [64] * 9, dtype=torch.int32, device=cuda)
    rows = torch.arange(e.numel(), dtype=torch.int32, device=cuda) % 30
    y = util.t2np_f32(layer.experts_grouped(x, e, rows))
    xh = util.t2np_f32(x)
    for a in (0, 69, 70, 72, 73, 82):
        ex = int(e[a])
        ref = oracle.expert_ffn(util.t2np_u32(w["gate_w"][ex]), util.t2np_bf16(w["gate_s"][ex]), util.t2np_u32(w["up_w"][ex]),
                                util.t2np_bf16(w["up_s"][ex]), util.t2np_u32(w["down_w"][ex]), util.t2np_bf16(w["down_s"][ex]),
                                xh[int(rows[a])], mode=0, round_out=True)
        util.assert_close(y[a], ref, "assignment %d" % a)
    layer.check()
    assert layer.experts_grouped(x, e[:0].contiguous(), rows[:0].contiguous()).shape == (0, hidden)
    with pytest.raises(lib.BlokError):
        layer.experts_grouped(x, torch.zeros(64 * 8 + 1, dtype=torch.int32, device=cuda))
    layer.close()
