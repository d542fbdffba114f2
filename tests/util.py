"""Shared helpers of the parity tests."""
import numpy as np
import torch

# Floating-point bar for outputs (fp32 accumulation, bf16 results) against the
# oracle's wide evaluation: max |a-b| / max |b| <= 2e-2 and cosine >= 0.9999.
MAX_ABS_REL = 2e-2
MIN_COSINE = 0.9999


def t2np_bf16(t):
    """torch bf16 tensor -> numpy uint16 bit patterns."""
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def t2np_f32(t):
    """torch bf16/f32 tensor -> numpy float32 values."""
    return t.detach().float().cpu().numpy()


def t2np_u32(t):
    return t.detach().contiguous().cpu().numpy().view(np.uint32)


def ids_np(t):
    """ids travel as int16 storage holding uint16 values."""
    return t.detach().contiguous().cpu().numpy().view(np.uint16)


def max_abs_rel(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    denom = np.max(np.abs(b))
    return float(np.max(np.abs(a - b)) / denom) if denom > 0 else float(np.max(np.abs(a - b)))


def cosine(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    na, nb = np.linalg.norm(a), np.linalg.norm(b)
    if na == 0 and nb == 0:
        return 1.0
    return float(a @ b / (na * nb))


def assert_close(actual, expected, what=""):
    r, c = max_abs_rel(actual, expected), cosine(actual, expected)
    assert r <= MAX_ABS_REL and c >= MIN_COSINE, "%s: max-abs-rel %.3e (bar %.0e), cosine %.6f (bar %.4f)" % (
        what, r, MAX_ABS_REL, c, MIN_COSINE)
    return r, c


def rand_i4(rng, rows, cols):
    """q ~ U{-8..7} and its packed words via plain numpy (independent of the oracle's packer)."""
    q = rng.integers(-8, 8, size=(rows, cols), dtype=np.int8)
    nib = (q.astype(np.int32) + 8).astype(np.uint32).reshape(rows, cols // 8, 8)
    w = np.zeros((rows, cols // 8), np.uint32)
    for k in range(8):
        w |= nib[:, :, k] << np.uint32(4 * k)
    return q, w


def rand_scales(rng, rows, groups, std=0.003):
    s = np.abs(rng.normal(0, std, size=(rows, groups))).astype(np.float32)
    return f32_to_bf16_np(s)


def f32_to_bf16_np(x):
    """round-to-nearest-even fp32 -> bf16 bit patterns, in numpy (independent of the oracle)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    return ((u + 0x7fff + lsb) >> 16).astype(np.uint16)


def bf16_np_to_f32(h):
    return (np.ascontiguousarray(h, np.uint16).astype(np.uint32) << 16).view(np.float32)


def np_bf16_to_torch(h, device):
    return torch.from_numpy(np.ascontiguousarray(h, np.uint16).view(np.int16)).to(device).view(torch.bfloat16)


def np_u32_to_torch(w, device):
    return torch.from_numpy(np.ascontiguousarray(w, np.uint32).view(np.int32)).to(device)


# ---- a materialised checkpoint in miniature: shard files plus the text index of scripts/model_fetch.py:113-127 ----

def checkpoint_tensors(cfg, get):
    """The tensors of the forward contract (src/kimi_exec.cu:736-778) for a model configuration, as
    (name, role, layer, expert, slot, dtype, shape, array) with the checkpoint's naming.  get(layer, model_name,
    dtype, shape) returns the numpy array of a model tensor; the router bias comes back fp32 and is stored as bf16."""
    H, c = cfg.hidden, cfg
    qk, kvo, lat = c.qk_nope + c.qk_rope, c.qk_nope + c.v_head, c.kv_rank + c.qk_rope
    out = []

    def bf(layer, role, slot, model_name, rows, cols=0):
        shape = (rows, cols) if cols else (rows,)
        prefix = "language_model.model.layers.%d." % layer if layer >= 0 else "language_model."
        out.append((prefix + slot + ".weight", role, layer, -1, slot, "bf16", shape, get(layer, model_name, np.uint16, shape)))

    for l in range(c.layers):
        bf(l, "attention_resident", "q_a_proj", "q_a_proj", c.q_rank, H)
        bf(l, "attention_resident", "q_a_layernorm", "q_a_layernorm", c.q_rank)
        bf(l, "attention_resident", "q_b_proj", "q_b_proj", c.heads * qk, c.q_rank)
        bf(l, "attention_resident", "kv_a_proj_with_mqa", "kv_a_proj_with_mqa", lat, H)
        bf(l, "attention_resident", "kv_a_layernorm", "kv_a_layernorm", c.kv_rank)
        bf(l, "attention_resident", "kv_b_proj", "kv_b_proj", c.heads * kvo, c.kv_rank)
        bf(l, "attention_resident", "o_proj", "o_proj", H, c.heads * c.v_head)
        bf(l, "resident", "input_layernorm", "input_layernorm", H)
        bf(l, "resident", "post_attention_layernorm", "post_attention_layernorm", H)
        if l < c.first_dense:
            bf(l, "dense_ffn_rowcol", "gate_proj", "gate_proj", c.dense_inter, H)
            bf(l, "dense_ffn_rowcol", "up_proj", "up_proj", c.dense_inter, H)
            bf(l, "dense_ffn_rowcol", "down_proj", "down_proj", H, c.dense_inter)
            continue
        bf(l, "router", "gate", "router", c.experts, H)
        bias = f32_to_bf16_np(get(l, "router_bias", np.float32, (c.experts,)))
        out.append(("language_model.model.layers.%d.mlp.gate.e_score_correction_bias" % l, "router", l, -1,
                    "e_score_correction_bias", "bf16", (c.experts,), bias))
        if c.shared_inter:
            bf(l, "shared_expert_resident", "gate_proj", "shared_gate", c.shared_inter, H)
            bf(l, "shared_expert_resident", "up_proj", "shared_up", c.shared_inter, H)
            bf(l, "shared_expert_resident", "down_proj", "shared_down", H, c.shared_inter)
        for proj, wn, sn, rows, cols in (("gate_proj", "gate_w", "gate_s", c.inter, H), ("up_proj", "up_w", "up_s", c.inter, H),
                                         ("down_proj", "down_w", "down_s", H, c.inter)):
            w = get(l, wn, np.uint32, (c.experts, rows, cols // 8))
            s = get(l, sn, np.uint16, (c.experts, rows, cols // 32))
            for e in range(c.experts):
                base = "language_model.model.layers.%d.mlp.experts.%d.%s." % (l, e, proj)
                out.append((base + "weight_packed", "routed_expert", l, e, proj + ".weight_packed", "i32", (rows, cols // 8), w[e]))
                out.append((base + "weight_scale", "routed_expert", l, e, proj + ".weight_scale", "bf16", (rows, cols // 32), s[e]))
    bf(-1, "resident", "embed_tokens", "embed_tokens", c.vocab, H)
    bf(-1, "resident", "norm", "norm", H)
    bf(-1, "resident", "lm_head", "lm_head", c.vocab, H)
    return out


def write_checkpoint(directory, tensors, shards=2, lead=8 + 1234):
    """Writes the tensors into `shards` files at unaligned offsets (a safetensors file starts with an 8-byte length and
    a JSON header) and returns the path of the runtime index describing them; 4 KiB-aligned read extents as the
    reference's materialize step computes them."""
    import os
    files = [open(os.path.join(directory, "model-%05d.safetensors" % i), "wb") for i in range(shards)]
    for f in files:
        f.write(b"\0" * lead)
    lines = ["blok-runtime-index-v1"]
    for i, (name, role, layer, expert, slot, dtype, shape, arr) in enumerate(tensors):
        f = files[i % shards]
        raw = np.ascontiguousarray(arr).tobytes()
        start = f.tell()
        f.write(raw)
        f.write(b"\0" * (3 + i % 5))  # neighbours are not aligned to anything
        off = start // 4096 * 4096
        end = (start + len(raw) + 4095) // 4096 * 4096
        lines.append("tensor %s %s %d %d %s %s %s %d %d 4096 %d %d %s" % (name, role, layer, expert, slot, dtype,
                                                                            "x".join(str(d) for d in shape), off, end - off, start,
                                                                            len(raw), f.name))
    for f in files:
        f.write(b"\0" * 4096)
        f.close()
    path = os.path.join(directory, "runtime-index.blok")
    with open(path, "w") as fh:
        fh.write("\n".join(lines) + "\n")
    return path
