"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (no dataset or checkpoint is involved):

  INT4 weights  q ~ Uniform{-8..7}, packed 8 nibbles per int32 (nibble = q + 8, low
                nibble = lowest column): a uniformly random 32-bit word IS eight
                independent uniform nibbles, so the packed tensor is drawn directly.
  scales        bf16 |N(0, 0.003)|
  bf16 weights  N(0, 0.006); router bias fp32 N(0, 0.01); activations bf16 N(0, 1).

Generation happens on the requested device with a torch.Generator seeded by
`seed`; parity tests copy the same bits to the host for the oracle.
"""
import torch

KIMI = dict(hidden=7168, inter=2048, experts=384, topk=8, shared_inter=2048, routed_scale=2.827,
            heads=64, qk_nope=128, qk_rope=64, v_head=128, q_rank=1536, kv_rank=512, vocab=163840,
            dense_inter=18432, layers=61, rope_theta=50000.0, rms_eps=1e-5)


def _gen(device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def packed_i4(shape_words, g, device):
    """int32 tensor of uniformly random words (= uniform nibbles)."""
    lo = torch.randint(0, 1 << 16, shape_words, generator=g, device=device, dtype=torch.int32)
    hi = torch.randint(0, 1 << 16, shape_words, generator=g, device=device, dtype=torch.int32)
    return lo | (hi << 16)


def scales(shape, g, device, std=0.003):
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).abs().to(torch.bfloat16)


def normal_bf16(shape, g, device, std):
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).to(torch.bfloat16)


def expert_weights(n, hidden, inter, g, device):
    """Expert-major INT4 arrays for n experts."""
    return dict(
        gate_w=packed_i4((n, inter, hidden // 8), g, device), gate_s=scales((n, inter, hidden // 32), g, device),
        up_w=packed_i4((n, inter, hidden // 8), g, device), up_s=scales((n, inter, hidden // 32), g, device),
        down_w=packed_i4((n, hidden, inter // 8), g, device), down_s=scales((n, hidden, inter // 32), g, device),
    )


def moe_layer_weights(device, seed=1, hidden=7168, inter=2048, experts=384, shared_inter=2048, experts_local=None):
    """Config-1 layer: router, INT4 routed experts, bf16 shared expert."""
    g = _gen(device, seed)
    n = experts if experts_local is None else experts_local
    w = dict(router_w=normal_bf16((experts, hidden), g, device, 0.006),
             router_bias=torch.randn(experts, generator=g, device=device, dtype=torch.float32) * 0.01)
    w.update(expert_weights(n, hidden, inter, g, device))
    if shared_inter:
        w.update(shared_gate=normal_bf16((shared_inter, hidden), g, device, 0.006),
                 shared_up=normal_bf16((shared_inter, hidden), g, device, 0.006),
                 shared_down=normal_bf16((hidden, shared_inter), g, device, 0.006))
    return w


def activations(T, hidden, device, seed):
    return normal_bf16((T, hidden), _gen(device, seed + 7919), device, 1.0)


def moe_layer_bytes(hidden=7168, inter=2048, experts=384, topk=8, shared_inter=2048, distinct_experts=None):
    """Algorithmic bytes of one layer pass: the weights and scales every selected expert
    reads once, the router matrix and bias, and the shared expert."""
    per_expert = 3 * (inter * hidden // 2 + inter * hidden // 32 * 2)
    k = topk if distinct_experts is None else distinct_experts
    return k * per_expert + experts * hidden * 2 + experts * 4 + 3 * shared_inter * hidden * 2


def mla_weights(device, seed=3, hidden=7168, heads=64, qk_nope=128, qk_rope=64, v_head=128, q_rank=1536, kv_rank=512,
                std=0.006):
    """Config-3 attention block: every projection bf16 N(0, std), RMSNorm weights 1."""
    g = _gen(device, seed)
    one = lambda n: torch.ones(n, dtype=torch.bfloat16, device=device)
    return dict(q_a=normal_bf16((q_rank, hidden), g, device, std), q_a_ln=one(q_rank),
                q_b=normal_bf16((heads * (qk_nope + qk_rope), q_rank), g, device, std),
                kv_a=normal_bf16((kv_rank + qk_rope, hidden), g, device, std), kv_a_ln=one(kv_rank),
                kv_b=normal_bf16((heads * (qk_nope + v_head), kv_rank), g, device, std),
                o=normal_bf16((hidden, heads * v_head), g, device, std))


def latent_cache(B, ctx, device, seed=3, width=576):
    """bf16 [B, ctx, 576] ~ N(0, 1)."""
    return normal_bf16((B, ctx, width), _gen(device, seed + 104729), device, 1.0)
