"""Generates tests/golden/third_party.npz: known-answer vectors from the two upstream
packages the reference pins its semantics to (its README names compressed-tensors'
pack_quantized layout and the HF DeepSeek-V3 modelling code), produced by importing
those packages in the build container:

  compressed_tensors (0.15.0.1)  pack_to_int32 / unpack_from_int32 for 4-bit values
  transformers (5.5.0)           deepseek_v3: sigmoid top-k routing, YaRN inverse
                                 frequencies and mscale, interleaved RoPE

The oracle (oracle/blok_oracle.cpp) is checked against these vectors by
tests/test_oracle_golden.py; the GPU box needs neither package.

Run: python tests/golden/make_third_party_golden.py
"""
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def pack_vectors(out):
    from compressed_tensors.compressors.pack_quantized.helpers import pack_to_int32, unpack_from_int32
    g = torch.Generator().manual_seed(11)
    q = torch.randint(-8, 8, (24, 96), generator=g, dtype=torch.int8)
    q[0, :16] = torch.arange(-8, 8, dtype=torch.int8)  # the documented 0x76543210 / 0xfedcba98 pattern
    packed = pack_to_int32(q, 4)
    back = unpack_from_int32(packed, 4, q.shape)
    assert torch.equal(back, q)
    out["pack_q"] = q.numpy()
    out["pack_words"] = packed.numpy().view(np.uint32)


def router_vectors(out):
    from transformers.models.deepseek_v3.configuration_deepseek_v3 import DeepseekV3Config
    from transformers.models.deepseek_v3.modeling_deepseek_v3 import DeepseekV3MoE
    cfg = DeepseekV3Config(hidden_size=64, intermediate_size=32, moe_intermediate_size=16, n_routed_experts=48,
                           num_experts_per_tok=8, n_group=1, topk_group=1, n_shared_experts=1,
                           routed_scaling_factor=2.827, norm_topk_prob=True, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=4, vocab_size=128)
    torch.manual_seed(5)
    moe = DeepseekV3MoE(cfg).eval()
    with torch.no_grad():
        moe.gate.weight.copy_((torch.randn(48, 64) * 0.2).bfloat16().float())
        moe.gate.e_score_correction_bias.copy_(torch.randn(48) * 0.05)
        x = torch.randn(20, 64).bfloat16().float()
        logits = moe.gate(x)
        idx, w = moe.route_tokens_to_experts(logits)
    out["router_w"] = moe.gate.weight.detach().numpy().astype(np.float32)
    out["router_bias"] = moe.gate.e_score_correction_bias.detach().numpy().astype(np.float32)
    out["router_x"] = x.numpy()
    out["router_idx"] = idx.numpy().astype(np.int64)      # unsorted top-k (a set per token)
    out["router_wts"] = w.numpy().astype(np.float32)


def yarn_vectors(out):
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    from transformers.models.deepseek_v3.configuration_deepseek_v3 import DeepseekV3Config
    from transformers.models.deepseek_v3.modeling_deepseek_v3 import apply_rotary_pos_emb_interleave, yarn_get_mscale
    for factor in (32.0, 64.0):
        cfg = DeepseekV3Config(hidden_size=64, num_attention_heads=1, qk_rope_head_dim=64, num_hidden_layers=1,
                               max_position_embeddings=int(4096 * factor),
                               rope_parameters=dict(rope_type="yarn", rope_theta=50000.0, factor=factor,
                                                    original_max_position_embeddings=4096, beta_fast=32.0,
                                                    beta_slow=1.0, mscale=1.0, mscale_all_dim=1.0))
        cfg.head_dim = 64
        inv_freq, attn_factor = ROPE_INIT_FUNCTIONS["yarn"](cfg, "cpu")
        tag = str(int(factor))
        out["yarn_inv_freq_" + tag] = inv_freq.numpy().astype(np.float32)
        out["yarn_attn_factor_" + tag] = np.float32(attn_factor)
        out["yarn_mscale_" + tag] = np.float32(yarn_get_mscale(factor, 1.0))
    # interleaved RoPE on one vector at one position, fp32 (no bf16 rounding points)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(1, 1, 1, 64, generator=g)
    pos = 1234
    ang = pos * torch.from_numpy(out["yarn_inv_freq_32"]).double()
    cos = torch.cat([ang.cos(), ang.cos()]).float()[None, None, :]
    sin = torch.cat([ang.sin(), ang.sin()]).float()[None, None, :]
    q, _ = apply_rotary_pos_emb_interleave(x, x.clone(), cos, sin)
    out["rope_x"] = x.reshape(64).numpy()
    out["rope_pos"] = np.int32(pos)
    out["rope_y"] = q.reshape(64).numpy()


if __name__ == "__main__":
    out = {}
    pack_vectors(out)
    router_vectors(out)
    yarn_vectors(out)
    path = os.path.join(HERE, "third_party.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")
    for k, v in out.items():
        print(" ", k, np.asarray(v).shape, np.asarray(v).dtype)
