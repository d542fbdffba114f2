"""GPU parity of the batch-1 routed-MoE decode layer (config 1) against the oracle."""
import numpy as np
import pytest
import torch

import util

pytestmark = pytest.mark.gpu


def _host_layer(w, chosen):
    """Copy router, shared expert and the chosen experts to the host for the oracle."""
    experts = w["router_w"].shape[0]
    slot_of = np.full(experts, -1, np.int32)
    chosen = sorted(set(int(e) for e in chosen))
    for i, e in enumerate(chosen):
        slot_of[e] = i
    idx = torch.tensor(chosen, device=w["gate_w"].device)
    packs = {k: util.t2np_u32(w[k].index_select(0, idx)) for k in ("gate_w", "up_w", "down_w")}
    scs = {k: util.t2np_bf16(w[k].index_select(0, idx)) for k in ("gate_s", "up_s", "down_s")}
    shared = [util.t2np_bf16(w[k]) if w.get(k) is not None else None for k in ("shared_gate", "shared_up", "shared_down")]
    return slot_of, packs, scs, shared


def _check(cuda, oracle, hidden, inter, experts, shared_inter, seed, topk=8):
    from blok_b200 import lib, synth
    w = synth.moe_layer_weights(cuda, seed=seed, hidden=hidden, inter=inter, experts=experts, shared_inter=shared_inter)
    if hidden < 7168:  # keep small layers in a comparable numeric range
        for k in ("gate_s", "up_s", "down_s"):
            w[k] = (w[k].float() * 8).bfloat16()
    layer = lib.MoeLayer(w, topk=topk, routed_scale=2.827)
    x = synth.activations(1, hidden, cuda, seed)[0].contiguous()
    y, ids, wts = layer.decode(x, return_routing=True)
    torch.cuda.synchronize()
    ids_h = util.ids_np(ids)
    xh = util.t2np_f32(x)
    oid, owt, margin, _ = oracle.router(util.t2np_bf16(w["router_w"]), util.t2np_f32(w["router_bias"]), xh[None], topk=topk,
                                        mode=0)
    if margin[0] > 2e-6:
        assert ids_h.tolist() == oid[0].tolist(), "top-k ids must be bit-exact"
    slot_of, packs, scs, shared = _host_layer(w, list(ids_h) + list(oid[0]))
    out, _, _ = oracle.moe_layer(util.t2np_bf16(w["router_w"]), util.t2np_f32(w["router_bias"]), slot_of, packs["gate_w"],
                                 scs["gate_s"], packs["up_w"], scs["up_s"], packs["down_w"], scs["down_s"], shared[0],
                                 shared[1], shared[2], xh[None], topk=topk, mode=0)
    r, c = util.assert_close(util.t2np_f32(y), out[0], "moe_decode")
    out1, _, _ = oracle.moe_layer(util.t2np_bf16(w["router_w"]), util.t2np_f32(w["router_bias"]), slot_of, packs["gate_w"],
                                  scs["gate_s"], packs["up_w"], scs["up_s"], packs["down_w"], scs["down_s"], shared[0],
                                  shared[1], shared[2], xh[None], topk=topk, mode=1)
    util.assert_close(util.t2np_f32(y), out1[0], "moe_decode vs ref_exact")
    np.testing.assert_allclose(util.t2np_f32(wts), owt[0], rtol=2e-5)
    y2 = layer.decode(x)
    assert torch.equal(y, y2), "decode must be deterministic"
    layer.close()
    return r, c


@pytest.mark.parametrize("impl", ["fused", "multi"])
@pytest.mark.parametrize("hidden,inter,experts,shared_inter,seed", [(512, 256, 16, 256, 11), (1024, 512, 32, 0, 12),
                                                                    (7168, 2048, 24, 2048, 13), (256, 256, 48, 32, 14)])
def test_moe_decode_small(cuda, oracle, monkeypatch, impl, hidden, inter, experts, shared_inter, seed):
    """Both implementations of the layer: the single persistent kernel and the multi-kernel path."""
    monkeypatch.setenv("BLOK_MOE_DECODE_IMPL", impl)
    _check(cuda, oracle, hidden, inter, experts, shared_inter, seed)


def test_moe_decode_many_tokens_fused(cuda, oracle):
    """Back-to-back launches on one handle: the kernel's self-cleaning counters must leave no state behind."""
    from blok_b200 import lib, synth
    w = synth.moe_layer_weights(cuda, seed=21, hidden=1024, inter=512, experts=32, shared_inter=512)
    layer = lib.MoeLayer(w)
    xs = synth.activations(24, 1024, cuda, 21)
    first = [layer.decode(xs[i]).clone() for i in range(24)]
    again = [layer.decode(xs[i]).clone() for i in range(24)]
    for a, b in zip(first, again):
        assert torch.equal(a, b)
    assert lib.load().blok_moe_layer_check(layer._handle, None) == 0
    layer.close()


def test_moe_decode_config1_full_size(cuda, oracle):
    """Config 1: 384 experts (9.5 GB packed), hidden 7168, shared expert, seed 1."""
    r, c = _check(cuda, oracle, 7168, 2048, 384, 2048, seed=1)
    print("config 1: max-abs-rel %.2e cosine %.7f" % (r, c))


def test_moe_decode_rejects_partial_expert_set(cuda):
    from blok_b200 import lib, synth
    w = synth.moe_layer_weights(cuda, seed=3, hidden=256, inter=256, experts=16, shared_inter=0, experts_local=8)
    layer = lib.MoeLayer(w)
    assert not layer.has_partial()       # no shared expert: the share's output rows would have no finisher
    with pytest.raises(lib.BlokError) as e:
        layer.decode(torch.zeros(256, dtype=torch.bfloat16, device=cuda))
    assert e.value.code == -7


@pytest.mark.parametrize("hidden,inter,experts,shared_inter,cuts", [(1024, 512, 32, 512, (0, 8, 32)), (512, 256, 16, 256, (0, 4, 9, 16)),
                                                                    (7168, 2048, 32, 2048, (0, 12, 32))])
def test_moe_decode_partial_shares_add_up(cuda, hidden, inter, experts, shared_inter, cuts):
    """blok_moe_decode_partial on handles that each hold a range of the experts: every handle reports the whole layer's
    routing and the same shared-expert output, and the shares, summed in fp32, rounded and added to the shared expert's
    output, give blok_moe_decode's result (equal up to the order of the fp32 sum of the slots: a last place of bf16).
    Many tokens in a row on the same handles: the number of slots a share runs changes from launch to launch (0 included),
    which is what its launch-spanning counters must survive."""
    from blok_b200 import lib, synth
    w = synth.moe_layer_weights(cuda, seed=31, hidden=hidden, inter=inter, experts=experts, shared_inter=shared_inter)
    whole = lib.MoeLayer(w)
    shares = []
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        ws = dict(w)
        for k in ("gate_w", "gate_s", "up_w", "up_s", "down_w", "down_s"):
            ws[k] = w[k][lo:hi].contiguous()
        shares.append(lib.MoeLayer(ws, expert_base=lo))
        assert shares[-1].has_partial()
    xs = synth.activations(40, hidden, cuda, 31)
    slots_seen = set()
    for i in range(40):
        y, ids, wts = whole.decode(xs[i], return_routing=True)
        total = torch.zeros(hidden, dtype=torch.float32, device=cuda)
        for (lo, hi), sh in zip(zip(cuts[:-1], cuts[1:]), shares):
            part, shared, pid, pwt = sh.decode_partial(xs[i], return_routing=True)
            assert torch.equal(pid, ids) and torch.equal(pwt, wts)
            total += part
            n_mine = int(((ids.int() & 0xFFFF) >= lo).sum() - ((ids.int() & 0xFFFF) >= hi).sum())
            slots_seen.add(n_mine)
            if n_mine == 0:
                assert torch.count_nonzero(part) == 0
        got = (total.bfloat16().float() + shared.float()).bfloat16()
        diff = (got.float() - y.float()).abs()
        assert float((diff / y.float().abs().clamp_min(1e-3)).max()) < 2 ** -6, i
        assert float((got == y).float().mean()) > 0.9, i
    for sh in shares:
        sh.check()
        sh.close()
    whole.check()
    whole.close()
    assert len(slots_seen) > 2, slots_seen
