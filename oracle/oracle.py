"""ctypes front end of the CPU oracle (oracle/blok_oracle.cpp).

Test infrastructure: imported only by tests/, by __graft_entry__.smoke() and by the
cpu-baseline / reference legs of bench.py.  The product package never imports it.

All arrays are numpy, C-contiguous.  bf16 tensors travel as uint16 bit patterns;
"activation" arrays are float32 holding bf16-representable values, which is the
reference's own convention (src/kimi_exec.cu:162-174, :240-241).
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
WIDE, REF_EXACT = 0, 1

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "libblok_oracle.so")
        if not os.path.exists(path):
            import importlib.util
            spec = importlib.util.spec_from_file_location("_blok_oracle_build", os.path.join(HERE, "build.py"))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build_oracle()
        _lib = C.CDLL(path)
        _lib.orc_num_threads.restype = C.c_int
        _lib.orc_yarn_mscale.restype = C.c_float
        _lib.orc_yarn_mscale.argtypes = [C.c_float, C.c_float]
        _lib.orc_lm_head_argmax.restype = C.c_uint32
        _lib.orc_moe_layer.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


def num_threads():
    return lib().orc_num_threads()


def set_num_threads(n):
    lib().orc_set_num_threads(C.c_int(n))


def f32_to_bf16(x):
    x = _c(x, np.float32)
    y = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16(_p(x), _p(y), C.c_long(x.size))
    return y


def bf16_to_f32(x):
    x = _c(x, np.uint16)
    y = np.empty(x.shape, np.float32)
    lib().orc_bf16_to_f32(_p(x), _p(y), C.c_long(x.size))
    return y


def bf16_round(x):
    return bf16_to_f32(f32_to_bf16(x))


def i4_pack(q):
    q = _c(q, np.int8)
    rows, cols = q.shape
    w = np.empty((rows, cols // 8), np.uint32)
    lib().orc_i4_pack(_p(q), _p(w), C.c_int(rows), C.c_int(cols))
    return w


def i4_dequant(w, scale):
    w = _c(w, np.uint32)
    scale = _c(scale, np.uint16)
    rows, cols = w.shape[0], w.shape[1] * 8
    out = np.empty((rows, cols), np.uint16)
    lib().orc_i4_dequant(_p(w), _p(scale), _p(out), C.c_int(rows), C.c_int(cols))
    return out


def i4_gemv(w, scale, x, mode=WIDE, round_out=True):
    w = _c(w, np.uint32)
    scale = _c(scale, np.uint16)
    x = _c(x, np.float32)
    rows, cols = w.shape[0], w.shape[1] * 8
    y = np.empty(rows, np.float32)
    lib().orc_i4_gemv(_p(w), _p(scale), _p(x), _p(y), C.c_int(rows), C.c_int(cols), C.c_int(mode), C.c_int(int(round_out)))
    return y


def bf16_gemv(w, x, mode=WIDE, round_out=True):
    w = _c(w, np.uint16)
    x = _c(x, np.float32)
    rows, cols = w.shape
    y = np.empty(rows, np.float32)
    lib().orc_bf16_gemv(_p(w), _p(x), _p(y), C.c_int(rows), C.c_int(cols), C.c_int(mode), C.c_int(int(round_out)))
    return y


def silu_mul(a, b, mode=WIDE):
    a = _c(a, np.float32)
    b = _c(b, np.float32)
    y = np.empty_like(a)
    lib().orc_silu_mul(_p(a), _p(b), _p(y), C.c_int(a.size), C.c_int(mode))
    return y


def rmsnorm(x, w, eps=1e-5, mode=WIDE):
    x = _c(x, np.float32)
    w = _c(w, np.uint16)
    y = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(w), _p(y), C.c_int(x.size), C.c_float(eps), C.c_int(mode))
    return y


def router(wr, bias, x, topk=8, routed_scale=2.827, mode=WIDE):
    """x [T, hidden] float32.  Returns ids [T,topk] uint16, wts [T,topk] f32, margin [T], scores [T,E]."""
    wr = _c(wr, np.uint16)
    bias = _c(bias, np.float32)
    x = _c(x, np.float32).reshape(-1, wr.shape[1])
    T, experts, hidden = x.shape[0], wr.shape[0], wr.shape[1]
    ids = np.empty((T, topk), np.uint16)
    wts = np.empty((T, topk), np.float32)
    margin = np.empty(T, np.float32)
    scores = np.empty((T, experts), np.float32)
    lib().orc_router(_p(wr), _p(bias), _p(x), C.c_int(T), C.c_int(experts), C.c_int(hidden), C.c_int(topk),
                     C.c_float(routed_scale), _p(ids), _p(wts), _p(margin), _p(scores), C.c_int(mode))
    return ids, wts, margin, scores


def expert_ffn(gw, gs, uw, us, dw, ds, x, mode=WIDE, round_out=True):
    gw, uw, dw = (_c(a, np.uint32) for a in (gw, uw, dw))
    gs, us, ds = (_c(a, np.uint16) for a in (gs, us, ds))
    x = _c(x, np.float32)
    inter, hidden = gw.shape[0], gw.shape[1] * 8
    y = np.empty(hidden, np.float32)
    lib().orc_expert_ffn(_p(gw), _p(gs), _p(uw), _p(us), _p(dw), _p(ds), _p(x), _p(y), C.c_int(hidden), C.c_int(inter),
                         C.c_int(mode), C.c_int(int(round_out)))
    return y


def bf16_mlp(gw, uw, dw, x, mode=WIDE, round_out=True):
    gw, uw, dw = (_c(a, np.uint16) for a in (gw, uw, dw))
    x = _c(x, np.float32)
    ffn, hidden = gw.shape
    y = np.empty(hidden, np.float32)
    lib().orc_bf16_mlp(_p(gw), _p(uw), _p(dw), _p(x), _p(y), C.c_int(hidden), C.c_int(ffn), C.c_int(mode),
                       C.c_int(int(round_out)))
    return y


def moe_layer(wr, bias, slot_of, gw, gs, uw, us, dw, ds, sgw, suw, sdw, x, topk=8, routed_scale=2.827, mode=WIDE):
    """Expert arrays are compact [n, out, in/8] / [n, out, in/32]; slot_of[e] indexes them (-1 = absent).

    Returns (out [T, hidden] f32, ids, wts); raises if routing hits an absent expert."""
    wr = _c(wr, np.uint16)
    bias = _c(bias, np.float32)
    slot_of = _c(slot_of, np.int32)
    gw, uw, dw = (_c(a, np.uint32) for a in (gw, uw, dw))
    gs, us, ds = (_c(a, np.uint16) for a in (gs, us, ds))
    experts, hidden = wr.shape
    inter = gw.shape[1]
    x = _c(x, np.float32).reshape(-1, hidden)
    T = x.shape[0]
    shared_inter = 0
    if sgw is not None:
        sgw, suw, sdw = (_c(a, np.uint16) for a in (sgw, suw, sdw))
        shared_inter = sgw.shape[0]
    out = np.empty((T, hidden), np.float32)
    ids = np.empty((T, topk), np.uint16)
    wts = np.empty((T, topk), np.float32)
    rc = lib().orc_moe_layer(_p(wr), _p(bias), _p(slot_of), _p(gw), _p(gs), _p(uw), _p(us), _p(dw), _p(ds), _p(sgw),
                             _p(suw), _p(sdw), _p(x), _p(out), C.c_int(T), C.c_int(experts), C.c_int(hidden),
                             C.c_int(inter), C.c_int(shared_inter), C.c_int(topk), C.c_float(routed_scale), _p(ids),
                             _p(wts), C.c_int(mode))
    if rc != 0:
        raise RuntimeError("oracle moe_layer: routing selected an expert that was not materialised")
    return out, ids, wts


def yarn_inv_freq(rotary=64, theta=50000.0, factor=32.0, beta_fast=32.0, beta_slow=1.0, original_ctx=4096.0):
    f = np.empty(rotary // 2, np.float32)
    lib().orc_yarn_inv_freq(_p(f), C.c_int(rotary), C.c_float(theta), C.c_float(factor), C.c_float(beta_fast),
                            C.c_float(beta_slow), C.c_float(original_ctx))
    return f


def yarn_mscale(factor=32.0, mscale_all_dim=1.0):
    return float(lib().orc_yarn_mscale(C.c_float(factor), C.c_float(mscale_all_dim)))


def rope_table(inv_freq, pos):
    inv_freq = _c(inv_freq, np.float32)
    cs = np.empty(2 * inv_freq.size, np.float32)
    lib().orc_rope_table(_p(inv_freq), C.c_int(inv_freq.size), C.c_int(pos), _p(cs))
    return cs


def rope_vec(x, cs):
    x = _c(x, np.float32)
    cs = _c(cs, np.float32)
    y = np.empty_like(x)
    lib().orc_rope_vec(_p(x), _p(y), _p(cs), C.c_int(x.size))
    return y


class MlaDims(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("hidden", "heads", "qk_nope", "qk_rope", "v_head", "q_rank", "kv_rank")]


KIMI_MLA = dict(hidden=7168, heads=64, qk_nope=128, qk_rope=64, v_head=128, q_rank=1536, kv_rank=512)


def mla_project(dims, w_qa, qa_ln, w_qb, w_kva, kva_ln, n, pos, inv_freq, eps=1e-5, mode=WIDE):
    d = MlaDims(**dims)
    w_qa, qa_ln, w_qb, w_kva, kva_ln = (_c(a, np.uint16) for a in (w_qa, qa_ln, w_qb, w_kva, kva_ln))
    n = _c(n, np.float32)
    inv_freq = _c(inv_freq, np.float32)
    q = np.empty((d.heads, d.qk_nope + d.qk_rope), np.float32)
    latent = np.empty(d.kv_rank + d.qk_rope, np.float32)
    lib().orc_mla_project(C.byref(d), _p(w_qa), _p(qa_ln), _p(w_qb), _p(w_kva), _p(kva_ln), _p(n), C.c_int(pos),
                          _p(inv_freq), C.c_float(eps), _p(q), _p(latent), C.c_int(mode))
    return q, latent


def mla_attend_ref(dims, w_kvb, q, latents, softmax_mscale, mode=WIDE):
    d = MlaDims(**dims)
    w_kvb = _c(w_kvb, np.uint16)
    q = _c(q, np.float32)
    latents = _c(latents, np.float32)
    seq = latents.shape[0]
    out = np.empty(d.heads * d.v_head, np.float32)
    lib().orc_mla_attend_ref(C.byref(d), _p(w_kvb), _p(q), _p(latents), C.c_int(seq), C.c_float(softmax_mscale), _p(out),
                             C.c_int(mode))
    return out


def mla_attend_absorbed(dims, w_kvb, q, latents16, softmax_mscale):
    d = MlaDims(**dims)
    w_kvb = _c(w_kvb, np.uint16)
    q = _c(q, np.float32)
    latents16 = _c(latents16, np.uint16)
    seq = latents16.shape[0]
    out = np.empty(d.heads * d.v_head, np.float32)
    lib().orc_mla_attend_absorbed(C.byref(d), _p(w_kvb), _p(q), _p(latents16), C.c_int(seq), C.c_float(softmax_mscale),
                                  _p(out))
    return out


def lm_head_argmax(w, n, mode=WIDE):
    w = _c(w, np.uint16)
    n = _c(n, np.float32)
    best = C.c_float(0)
    tok = lib().orc_lm_head_argmax(_p(w), _p(n), C.c_int(w.shape[0]), C.c_int(w.shape[1]), C.c_int(mode), C.byref(best))
    return int(tok), float(best.value)


def add_round(a, b):
    a = _c(a, np.float32).copy()
    b = _c(b, np.float32)
    lib().orc_add_round(_p(a), _p(b), C.c_int(a.size))
    return a
