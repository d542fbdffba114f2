"""The whole decode step (config 4 in miniature) against a step composed from the oracle's functions."""
import numpy as np
import pytest
import torch

import util

pytestmark = pytest.mark.gpu

CFG = dict(layers=3, first_dense=1, hidden=1024, vocab=2048, dense_inter=512, inter=256, experts=16, topk=8,
           shared_inter=256, q_rank=256, max_batch=2, max_ctx=32, yarn_factor=64.0)


class OracleModel:
    """generate()'s per-token body (src/kimi_exec.cu:801-884) composed from oracle functions, batch 1."""

    def __init__(self, orc, model):
        self.o, c = orc, model.cfg
        self.c = c
        H, L = c.hidden, c.layers
        self.dims = dict(hidden=H, heads=c.heads, qk_nope=c.qk_nope, qk_rope=c.qk_rope, v_head=c.v_head, q_rank=c.q_rank,
                         kv_rank=c.kv_rank)
        t = lambda l, n, dt=np.uint16, sh=None: model.tensor(l, n, dt, sh)
        self.emb = t(-1, "embed_tokens", np.uint16, (c.vocab, H))
        self.norm = t(-1, "norm")
        self.head = t(-1, "lm_head", np.uint16, (c.vocab, H))
        self.layers = []
        qk, kvo, lat = c.qk_nope + c.qk_rope, c.qk_nope + c.v_head, c.kv_rank + c.qk_rope
        for l in range(L):
            w = dict(ln0=t(l, "input_layernorm"), ln1=t(l, "post_attention_layernorm"),
                     q_a=t(l, "q_a_proj", np.uint16, (c.q_rank, H)), q_a_ln=t(l, "q_a_layernorm"),
                     q_b=t(l, "q_b_proj", np.uint16, (c.heads * qk, c.q_rank)),
                     kv_a=t(l, "kv_a_proj_with_mqa", np.uint16, (lat, H)), kv_a_ln=t(l, "kv_a_layernorm"),
                     kv_b=t(l, "kv_b_proj", np.uint16, (c.heads * kvo, c.kv_rank)),
                     o=t(l, "o_proj", np.uint16, (H, c.heads * c.v_head)), rows=[])
            if l < c.first_dense:
                w.update(g=t(l, "gate_proj", np.uint16, (c.dense_inter, H)), u=t(l, "up_proj", np.uint16, (c.dense_inter, H)),
                         d=t(l, "down_proj", np.uint16, (H, c.dense_inter)))
            else:
                E, I, S = c.experts, c.inter, c.shared_inter
                w.update(router=t(l, "router", np.uint16, (E, H)), bias=t(l, "router_bias", np.float32),
                         gw=t(l, "gate_w", np.uint32, (E, I, H // 8)), gs=t(l, "gate_s", np.uint16, (E, I, H // 32)),
                         uw=t(l, "up_w", np.uint32, (E, I, H // 8)), us=t(l, "up_s", np.uint16, (E, I, H // 32)),
                         dw=t(l, "down_w", np.uint32, (E, H, I // 8)), ds=t(l, "down_s", np.uint16, (E, H, I // 32)),
                         sg=t(l, "shared_gate", np.uint16, (S, H)), su=t(l, "shared_up", np.uint16, (S, H)),
                         sd=t(l, "shared_down", np.uint16, (H, S)))
            self.layers.append(w)
        self.inv = orc.yarn_inv_freq(c.qk_rope, c.rope_theta, c.yarn_factor, c.yarn_beta_fast, c.yarn_beta_slow,
                                     c.yarn_original_ctx)
        self.ms = orc.yarn_mscale(c.yarn_factor, c.yarn_mscale_all_dim)
        self.pos = 0

    def step(self, tok):
        o, c = self.o, self.c
        x = util.bf16_np_to_f32(self.emb[tok])
        for l, w in enumerate(self.layers):
            n = o.rmsnorm(x, w["ln0"], c.rms_eps, mode=1)
            q, lat = o.mla_project(self.dims, w["q_a"], w["q_a_ln"], w["q_b"], w["kv_a"], w["kv_a_ln"], n, self.pos, self.inv,
                                   c.rms_eps, mode=1)
            w["rows"].append(util.f32_to_bf16_np(lat))
            av = o.mla_attend_absorbed(self.dims, w["kv_b"], q, np.stack(w["rows"]), self.ms)
            x = o.add_round(x, o.bf16_gemv(w["o"], av, mode=0, round_out=True))
            n = o.rmsnorm(x, w["ln1"], c.rms_eps, mode=1)
            if l < c.first_dense:
                f = o.bf16_mlp(w["g"], w["u"], w["d"], n, mode=0, round_out=True)
            else:
                f = o.moe_layer(w["router"], w["bias"], np.arange(c.experts, dtype=np.int32), w["gw"], w["gs"], w["uw"], w["us"],
                                w["dw"], w["ds"], w["sg"], w["su"], w["sd"], n[None], topk=c.topk, routed_scale=c.routed_scale,
                                mode=0)[0][0]
            x = o.add_round(x, f)
        n = o.rmsnorm(x, self.norm, c.final_rms_eps, mode=1)
        logits = o.bf16_gemv(self.head, n, mode=0, round_out=True)
        self.last_hidden = n        # the final-normed hidden state the sampler reads (:880-881)
        self.pos += 1
        order = np.argsort(-logits, kind="stable")
        return int(order[0]), float(logits[order[0]] - logits[order[1]]), x


def _sharpen(model):
    """Random-init logits are nearly flat; scale the router and the head so that routing and sampling are decisive."""
    c = model.cfg
    for l in range(c.first_dense, c.layers):
        r = util.bf16_np_to_f32(model.tensor(l, "router", np.uint16)) * 40
        model.write_tensor(l, "router", util.f32_to_bf16_np(r))
    h = util.bf16_np_to_f32(model.tensor(-1, "lm_head", np.uint16)) * 8
    model.write_tensor(-1, "lm_head", util.f32_to_bf16_np(h))


def test_model_steps_match_oracle(cuda, oracle):
    from blok_b200 import lib
    model = lib.Model(seed=4, **CFG)
    _sharpen(model)
    orc = OracleModel(oracle, model)
    tok, clear, total = 7, 0, 0
    ids = torch.tensor([tok], dtype=torch.int32, device=cuda)
    for step in range(6):
        nxt = model.step(ids)
        want, margin, _ = orc.step(int(ids[0]))
        got = int(nxt[0])
        total += 1
        if margin > 0.02:   # a bf16 logit step at this magnitude; closer calls may legitimately flip
            clear += 1
            assert got == want, "step %d: got %d want %d (margin %.3f)" % (step, got, want, margin)
        ids = torch.tensor([want], dtype=torch.int32, device=cuda)
    assert clear >= total - 2
    model.close()


def test_full_size_layers_and_full_vocabulary_match_oracle(cuda, oracle):
    """Config 4's shapes at full size, two layers deep (the dense layer and one MoE layer of 384 experts, hidden 7168,
    MLA with 64 heads, vocabulary 163840): three decode steps against the oracle's composition of the same layers.
    Checked per step: the final-normed hidden state (blok_model_hidden) and the greedy token over the whole vocabulary."""
    from blok_b200 import lib
    model = lib.Model(seed=4, layers=2, max_batch=1, max_ctx=16)
    _sharpen(model)
    orc = OracleModel(oracle, model)
    ids = torch.tensor([11], dtype=torch.int32, device=cuda)
    clear = 0
    for step in range(3):
        nxt = model.step(ids)
        got_hidden = util.t2np_f32(model.hidden(1))[0]
        want, margin, _ = orc.step(int(ids[0]))
        r, c = util.assert_close(got_hidden, util.bf16_np_to_f32(util.f32_to_bf16_np(orc.last_hidden)), "full-size hidden state, step %d" % step)
        if margin > 0.02:
            clear += 1
            assert int(nxt[0]) == want, "step %d: got %d want %d (margin %.3f)" % (step, int(nxt[0]), want, margin)
        print("step %d: hidden max-abs-rel %.2e cosine %.6f, token %d (oracle %d, margin %.3f)" % (step, r, c, int(nxt[0]), want, margin))
        ids = torch.tensor([want], dtype=torch.int32, device=cuda)
    assert clear >= 2
    model.check()
    model.close()


def test_generate_replays_prompt_and_stops(cuda, oracle):
    from blok_b200 import lib
    model = lib.Model(seed=5, **CFG)
    _sharpen(model)
    prompt = [3, 1, 4, 1, 5]
    a = model.generate(prompt, 6)
    b = model.generate(prompt, 6)
    assert a == b and 1 <= len(a) <= 6 and all(0 <= t < CFG["vocab"] for t in a)
    # batch-2 stepping of the same prompt gives the same first sample for both sequences
    model.reset()
    for t in prompt:
        nxt = model.step(torch.tensor([t, t], dtype=torch.int32, device=cuda))
    assert int(nxt[0]) == int(nxt[1]) == a[0]
    # the sequence budget is enforced like the reference's context check (:784)
    with pytest.raises(lib.BlokError):
        model.generate(prompt, CFG["max_ctx"])
    # eos stops generation before it is emitted
    model.cfg.eos_id = a[0]
    m2 = lib.Model(seed=5, **dict(CFG, eos_id=a[0]))
    _sharpen(m2)
    assert m2.generate(prompt, 6) == []
    m2.close()
    model.close()


def test_load_index_replaces_every_weight(cuda, tmp_path):
    """Model B (other seed) loads the checkpoint dumped from model A: every tensor equals A's, and B generates A's tokens."""
    from blok_b200 import lib
    a = lib.Model(seed=31, **CFG)
    b = lib.Model(seed=32, **CFG)
    prompt = [3, 1, 4, 1, 5]
    want = a.generate(prompt, 8)
    assert b.generate(prompt, 8) != want
    tensors = util.checkpoint_tensors(a.cfg, lambda l, n, dt, sh: a.tensor(l, n, dt, sh))
    path = util.write_checkpoint(str(tmp_path), tensors, shards=3)
    b.load_index(path)
    for l, name, dt in ((-1, "lm_head", np.uint16), (0, "down_proj", np.uint16), (1, "router_bias", np.float32),
                        (2, "gate_w", np.uint32), (2, "down_s", np.uint16), (1, "kv_b_proj", np.uint16)):
        ta, tb = a.tensor(l, name, dt), b.tensor(l, name, dt)
        if name == "router_bias":  # stored as bf16 in a checkpoint
            ta = util.bf16_np_to_f32(util.f32_to_bf16_np(ta))
        assert np.array_equal(ta, tb), (l, name)
    b.reset()
    got = b.generate(prompt, 8)
    # the router bias lost its low mantissa bits on the way through the checkpoint; A with the same bias must agree
    a.write_tensor(1, "router_bias", util.bf16_np_to_f32(util.f32_to_bf16_np(a.tensor(1, "router_bias", np.float32))))
    a.write_tensor(2, "router_bias", util.bf16_np_to_f32(util.f32_to_bf16_np(a.tensor(2, "router_bias", np.float32))))
    a.reset()
    assert got == a.generate(prompt, 8)
    a.close()
    b.close()


def test_sharded_model_holds_the_slices_of_the_unsharded_tensors(cuda, tmp_path):
    """Expert parallelism (config 4): rank r of w holds experts [r E/w, (r+1) E/w) of every MoE layer and everything else
    in full.  Its synthetic expert tensors are the slices of the unsharded model's, and the index loader reads into a
    shard only the experts the rank holds."""
    from blok_b200 import lib
    CFG = dict(globals()["CFG"], inter=512, shared_inter=512)      # the sizes the grouped expert kernels take
    full = lib.Model(seed=31, **CFG)
    c = full.cfg
    world = 4
    per = c.experts // world
    shapes = {"gate_w": (c.inter, c.hidden // 8), "down_w": (c.hidden, c.inter // 8), "up_s": (c.inter, c.hidden // 32)}
    other = lib.Model(seed=77, **CFG)
    path = util.write_checkpoint(str(tmp_path), util.checkpoint_tensors(other.cfg, lambda l, n, dt, sh: other.tensor(l, n, dt, sh)),
                                 shards=3)
    for rank in (0, 3):
        shard = lib.Model(seed=31, **dict(CFG, ep_rank=rank, ep_world=world))
        for name, sh in shapes.items():
            dt = np.uint32 if name.endswith("_w") else np.uint16
            want = full.tensor(2, name, dt, (c.experts,) + sh)[rank * per:(rank + 1) * per]
            assert np.array_equal(shard.tensor(2, name, dt, (per,) + sh), want), (rank, name)
        assert np.array_equal(shard.tensor(1, "router", np.uint16), full.tensor(1, "router", np.uint16))
        assert np.array_equal(shard.tensor(-1, "lm_head", np.uint16), full.tensor(-1, "lm_head", np.uint16))
        shard.load_index(path)          # the checkpoint of ANOTHER model: the shard must now hold that model's slices
        for name, sh in shapes.items():
            dt = np.uint32 if name.endswith("_w") else np.uint16
            want = other.tensor(1, name, dt, (c.experts,) + sh)[rank * per:(rank + 1) * per]
            assert np.array_equal(shard.tensor(1, name, dt, (per,) + sh), want), (rank, name)
        assert np.array_equal(shard.tensor(2, "kv_b_proj", np.uint16), other.tensor(2, "kv_b_proj", np.uint16))
        with pytest.raises(lib.BlokError) as e:          # no communicator yet: a step is refused, nothing is launched
            shard.step(torch.zeros(1, dtype=torch.int32, device=cuda))
        assert e.value.code == -4
        shard.close()
    with pytest.raises(lib.BlokError):
        lib.Model(seed=1, **dict(CFG, ep_rank=4, ep_world=4))
    full.close()
    other.close()


def test_a_wait_that_gave_up_in_a_layer_voids_the_generation(cuda):
    """The decode kernels' waits are bounded and leave an error word; generate() must not return tokens after one.
    The word is set from the host here (blok_moe_layer_debug_set_error): no wait is made to run out on the device."""
    import ctypes as C
    from blok_b200 import lib
    m = lib.Model(seed=5, **CFG)
    want = m.generate([3, 1, 4], 4)
    m.check()
    assert lib.load().blok_model_debug_set_layer_error(m._handle, C.c_int(1), C.c_uint(2), None) == 0
    with pytest.raises(lib.BlokError) as e:
        m.check()
    assert e.value.code == -5 and "layer 1" in str(e.value)
    m.check()                                   # reported once; the handle stays usable
    assert m.generate([3, 1, 4], 4) == want
    m.close()
