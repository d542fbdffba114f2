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
