"""ctypes front end of libblok_b200.so.

Each wrapper mirrors one host op of the reference executor (src/kimi_exec.cu) and
takes torch CUDA tensors; the tensor's data pointer and the current CUDA stream
are what crosses the C ABI.  A missing or stale library is an error, never a
fallback.
"""
import ctypes as C
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libblok_b200.so")

OK = 0
ABI_VERSION = 3  # BLOK_ABI_VERSION of include/blok_b200.h: the layout of the structures mirrored below


class BlokError(RuntimeError):
    def __init__(self, code, message):
        super().__init__("blok_b200 error %d: %s" % (code, message))
        self.code = code


class MoeWeights(C.Structure):
    _fields_ = [
        ("hidden", C.c_int), ("inter", C.c_int), ("experts", C.c_int), ("topk", C.c_int), ("shared_inter", C.c_int),
        ("routed_scale", C.c_float),
        ("router_w", C.c_void_p), ("router_bias", C.c_void_p),
        ("expert_base", C.c_int), ("experts_local", C.c_int),
        ("gate_w", C.c_void_p), ("gate_s", C.c_void_p), ("up_w", C.c_void_p), ("up_s", C.c_void_p),
        ("down_w", C.c_void_p), ("down_s", C.c_void_p),
        ("shared_gate", C.c_void_p), ("shared_up", C.c_void_p), ("shared_down", C.c_void_p),
    ]


_lib = None


def load():
    """Load the CUDA library; raises if it has not been built (python -m blok_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise BlokError(-100, "%s is missing: run `python -m blok_b200.build` (there is no CPU fallback)" % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    if lib.blok_abi_version() != ABI_VERSION:
        raise BlokError(-100, "%s has ABI version %d, this front end needs %d: rebuild with `python -m blok_b200.build --force`"
                        % (LIB_PATH, lib.blok_abi_version(), ABI_VERSION))
    lib.blok_last_error.restype = C.c_char_p
    lib.blok_kernel_launch_count.restype = C.c_longlong
    for name in ("blok_expert_ffn_workspace_bytes", "blok_bf16_mlp_workspace_bytes", "blok_router_workspace_bytes"):
        getattr(lib, name).restype = C.c_size_t
    _lib = lib
    return lib


def _check(rc):
    if rc != OK:
        raise BlokError(rc, load().blok_last_error().decode())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t, dtype=None, name="tensor"):
    if t is None:
        return C.c_void_p(0)
    if not t.is_cuda:
        raise BlokError(-1, "%s must be a CUDA tensor" % name)
    if not t.is_contiguous():
        raise BlokError(-1, "%s must be contiguous" % name)
    if dtype is not None and t.dtype != dtype:
        raise BlokError(-1, "%s must have dtype %s, got %s" % (name, dtype, t.dtype))
    return C.c_void_p(t.data_ptr())


def kernel_launch_count():
    """Kernels launched by the library so far in this process."""
    return int(load().blok_kernel_launch_count())


def i4_dequant(w_packed, scale):
    """bf16 [rows, cols] = bf16_rn(q * scale); the bit-exactness probe (src/kimi_exec.cu:311-312)."""
    rows, cols = w_packed.shape[0], w_packed.shape[1] * 8
    out = torch.empty((rows, cols), dtype=torch.bfloat16, device=w_packed.device)
    _check(load().blok_i4_dequant(_ptr(w_packed, torch.int32, "weight_packed"), _ptr(scale, torch.bfloat16, "weight_scale"),
                                  _ptr(out), C.c_int(rows), C.c_int(cols), _stream()))
    return out


def i4_gemv(w_packed, scale, x):
    """matvec_i4_slice (src/kimi_exec.cu:688): y[rows] from x[cols]; bf16 in/out, or the fp32 shim if x is fp32."""
    rows, cols = w_packed.shape[0], w_packed.shape[1] * 8
    if x.numel() != cols:
        raise BlokError(-2, "x has %d elements, expected %d" % (x.numel(), cols))
    y = torch.empty(rows, dtype=x.dtype, device=x.device)
    if x.dtype == torch.float32:
        _check(load().blok_i4_gemv_f32(_ptr(w_packed, torch.int32), _ptr(scale, torch.bfloat16), _ptr(x), _ptr(y),
                                       C.c_int(rows), C.c_int(cols), _stream()))
    else:
        _check(load().blok_i4_gemv(_ptr(w_packed, torch.int32), _ptr(scale, torch.bfloat16), _ptr(x, torch.bfloat16), _ptr(y),
                                   C.c_int(rows), C.c_int(cols), _stream()))
    return y


def expert_ffn(gate_w, gate_s, up_w, up_s, down_w, down_s, x, workspace=None):
    """One routed expert, y = down(SiLU(gate x) * up x) (src/kimi_exec.cu:853-869)."""
    inter, hidden = gate_w.shape[0], gate_w.shape[1] * 8
    lib = load()
    need = lib.blok_expert_ffn_workspace_bytes(C.c_int(hidden), C.c_int(inter))
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    y = torch.empty(hidden, dtype=torch.bfloat16, device=x.device)
    _check(lib.blok_expert_ffn(_ptr(gate_w, torch.int32), _ptr(gate_s, torch.bfloat16), _ptr(up_w, torch.int32),
                               _ptr(up_s, torch.bfloat16), _ptr(down_w, torch.int32), _ptr(down_s, torch.bfloat16),
                               _ptr(x, torch.bfloat16), _ptr(y), C.c_int(hidden), C.c_int(inter), _ptr(workspace),
                               C.c_size_t(workspace.numel() * workspace.element_size()), _stream()))
    return y


def expert_ffn_static(gate_w, gate_s, up_w, up_s, down_w, down_s, x, out=None):
    """One routed expert without a workspace argument: the intermediate vector lives in a fixed array inside the
    library, so the call allocates nothing on the device when `out` is given.  For callers that may not allocate;
    inter is limited to blok_expert_ffn_static_max_inter(); calls that can overlap on the GPU race on that array."""
    inter, hidden = gate_w.shape[0], gate_w.shape[1] * 8
    y = torch.empty(hidden, dtype=torch.bfloat16, device=x.device) if out is None else out
    _check(load().blok_expert_ffn_static(_ptr(gate_w, torch.int32), _ptr(gate_s, torch.bfloat16), _ptr(up_w, torch.int32),
                                         _ptr(up_s, torch.bfloat16), _ptr(down_w, torch.int32),
                                         _ptr(down_s, torch.bfloat16), _ptr(x, torch.bfloat16), _ptr(y, torch.bfloat16),
                                         C.c_int(hidden), C.c_int(inter), _stream()))
    return y


def bf16_gemv(w, x, out_f32=False):
    """matvec_bf16_k / matvec_bf16_f32_k (src/kimi_exec.cu:272-298) for x [T<=8, cols] or [cols]."""
    rows, cols = w.shape
    x2 = x.reshape(-1, cols)
    T = x2.shape[0]
    y = torch.empty((T, rows), dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    _check(load().blok_bf16_gemv(_ptr(w, torch.bfloat16), _ptr(x2, torch.bfloat16), _ptr(None if out_f32 else y),
                                 _ptr(y if out_f32 else None), C.c_int(rows), C.c_int(cols), C.c_int(T), _stream()))
    return y.reshape(*x.shape[:-1], rows)


def bf16_mlp(gate, up, down, x):
    """bf16_mlp (src/kimi_exec.cu:674-686) without the running-sum side effect."""
    ffn, hidden = gate.shape
    x2 = x.reshape(-1, hidden)
    T = x2.shape[0]
    lib = load()
    need = lib.blok_bf16_mlp_workspace_bytes(C.c_int(hidden), C.c_int(ffn), C.c_int(T))
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=x.device)
    y = torch.empty((T, hidden), dtype=torch.bfloat16, device=x.device)
    _check(lib.blok_bf16_mlp(_ptr(gate, torch.bfloat16), _ptr(up, torch.bfloat16), _ptr(down, torch.bfloat16),
                             _ptr(x2, torch.bfloat16), _ptr(y), C.c_int(hidden), C.c_int(ffn), C.c_int(T), _ptr(ws),
                             C.c_size_t(ws.numel()), _stream()))
    return y.reshape(x.shape)


def rmsnorm(x, w, eps=1e-5, out=None):
    """rmsnorm_k (src/kimi_exec.cu:258-270); x [T, n] or [n]."""
    n = x.shape[-1]
    T = x.numel() // n if n else 0
    y = torch.empty_like(x) if out is None else out
    _check(load().blok_rmsnorm(_ptr(x, torch.bfloat16), _ptr(w, torch.bfloat16), _ptr(y, torch.bfloat16), C.c_int(T),
                               C.c_int(n), C.c_float(eps), _stream()))
    return y



def add_rmsnorm(x, t, w, eps=1e-5):
    """x <- bf16(x + t) in place, returns RMSNorm(x) * w (one launch: src/kimi_exec.cu:248-251 then :258-270)."""
    n = x.shape[-1]
    T = x.numel() // n if n else 0
    y = torch.empty_like(x)
    _check(load().blok_add_rmsnorm(_ptr(x, torch.bfloat16), _ptr(t, torch.bfloat16), _ptr(w, torch.bfloat16), _ptr(y, torch.bfloat16),
                                   C.c_int(T), C.c_int(n), C.c_float(eps), _stream()))
    return y

def add_(a, b):
    """a = bf16(a + b), add_k (src/kimi_exec.cu:248-251)."""
    _check(load().blok_add_bf16(_ptr(a, torch.bfloat16), _ptr(b, torch.bfloat16), C.c_long(a.numel()), _stream()))
    return a


def router(router_w, bias, x, topk=8, routed_scale=2.827):
    """Router (src/kimi_exec.cu:836-842): returns ids uint16 [T, topk] (as int16 storage) and weights fp32 [T, topk]."""
    experts, hidden = router_w.shape
    x2 = x.reshape(-1, hidden)
    T = x2.shape[0]
    lib = load()
    need = lib.blok_router_workspace_bytes(C.c_int(T), C.c_int(experts))
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=x.device)
    ids = torch.empty((T, topk), dtype=torch.int16, device=x.device)
    wts = torch.empty((T, topk), dtype=torch.float32, device=x.device)
    _check(lib.blok_router(_ptr(router_w, torch.bfloat16), _ptr(bias, torch.float32), _ptr(x2, torch.bfloat16), C.c_int(T),
                           C.c_int(experts), C.c_int(hidden), C.c_int(topk), C.c_float(routed_scale), _ptr(ids), _ptr(wts),
                           _ptr(ws), C.c_size_t(ws.numel()), _stream()))
    return ids, wts


def moe_combine(y_assign, wts, shared=None):
    """out[t] = bf16(bf16(sum_k w[t,k] * y[t*topk+k]) + shared[t]) (src/kimi_exec.cu:399-407, :248)."""
    T, topk = wts.shape
    hidden = y_assign.shape[-1]
    out = torch.empty((T, hidden), dtype=torch.bfloat16, device=y_assign.device)
    _check(load().blok_moe_combine(_ptr(y_assign, torch.bfloat16), _ptr(wts, torch.float32), _ptr(shared, torch.bfloat16),
                                   C.c_int(T), C.c_int(topk), C.c_int(hidden), _ptr(out), _stream()))
    return out


class MoeLayer:
    """Handle of one routed-MoE layer (the MoE branch of src/kimi_exec.cu:836-875).

    `weights` is a dict of CUDA tensors:
      router_w bf16 [E, H], router_bias f32 [E],
      gate_w/up_w int32 [n, I, H/8], gate_s/up_s bf16 [n, I, H/32],
      down_w int32 [n, H, I/8], down_s bf16 [n, H, I/32],
      optional shared_gate/shared_up bf16 [S, H], shared_down bf16 [H, S].
    The tensors are borrowed: this object keeps references so they outlive the handle.
    """

    def __init__(self, weights, topk=8, routed_scale=2.827, expert_base=0, max_tokens=1):
        self.weights = dict(weights)
        w = self.weights
        E, H = w["router_w"].shape
        n, I = w["gate_w"].shape[0], w["gate_w"].shape[1]
        S = w["shared_gate"].shape[0] if w.get("shared_gate") is not None else 0
        self.hidden, self.inter, self.experts, self.topk, self.shared_inter = H, I, E, topk, S
        self.experts_local, self.expert_base = n, expert_base
        mw = MoeWeights(
            hidden=H, inter=I, experts=E, topk=topk, shared_inter=S, routed_scale=routed_scale,
            router_w=_ptr(w["router_w"], torch.bfloat16, "router_w").value,
            router_bias=_ptr(w["router_bias"], torch.float32, "router_bias").value,
            expert_base=expert_base, experts_local=n,
            gate_w=_ptr(w["gate_w"], torch.int32, "gate_w").value, gate_s=_ptr(w["gate_s"], torch.bfloat16, "gate_s").value,
            up_w=_ptr(w["up_w"], torch.int32, "up_w").value, up_s=_ptr(w["up_s"], torch.bfloat16, "up_s").value,
            down_w=_ptr(w["down_w"], torch.int32, "down_w").value, down_s=_ptr(w["down_s"], torch.bfloat16, "down_s").value,
            shared_gate=_ptr(w.get("shared_gate"), torch.bfloat16).value,
            shared_up=_ptr(w.get("shared_up"), torch.bfloat16).value,
            shared_down=_ptr(w.get("shared_down"), torch.bfloat16).value,
        )
        self._handle = C.c_void_p()
        self.device = w["router_w"].device
        with torch.cuda.device(self.device):
            _check(load().blok_moe_layer_create(C.byref(mw), C.c_int(max_tokens), C.byref(self._handle)))
        self.max_tokens = max_tokens

    def close(self):
        if getattr(self, "_handle", None) is not None and self._handle.value:
            load().blok_moe_layer_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def decode(self, x, out=None, return_routing=False):
        """Batch-1 decode layer: x bf16 [hidden] -> y bf16 [hidden]."""
        y = torch.empty(self.hidden, dtype=torch.bfloat16, device=x.device) if out is None else out
        ids = wts = None
        if return_routing:
            ids = torch.empty(self.topk, dtype=torch.int16, device=x.device)
            wts = torch.empty(self.topk, dtype=torch.float32, device=x.device)
        _check(load().blok_moe_decode(self._handle, _ptr(x, torch.bfloat16, "x"), _ptr(y, torch.bfloat16, "y"), _ptr(ids),
                                      _ptr(wts), _stream()))
        return (y, ids, wts) if return_routing else y

    def has_partial(self):
        return bool(load().blok_moe_layer_has_partial(self._handle))

    def decode_partial(self, x, return_routing=False):
        """A rank's share of the batch-1 layer (blok_moe_decode_partial): x bf16 [hidden] -> (part fp32 [hidden], the
        weighted sum of the selected experts this handle holds; shared bf16 [hidden], the shared expert's output)."""
        part = torch.empty(self.hidden, dtype=torch.float32, device=x.device)
        shared = torch.empty(self.hidden, dtype=torch.bfloat16, device=x.device)
        ids = wts = None
        if return_routing:
            ids = torch.empty(self.topk, dtype=torch.int16, device=x.device)
            wts = torch.empty(self.topk, dtype=torch.float32, device=x.device)
        _check(load().blok_moe_decode_partial(self._handle, _ptr(x, torch.bfloat16, "x"), _ptr(part), _ptr(shared), _ptr(ids),
                                              _ptr(wts), _stream()))
        return (part, shared, ids, wts) if return_routing else (part, shared)

    def batched(self, x, return_routing=False):
        """Batched layer (config 2): x bf16 [T, hidden] -> y bf16 [T, hidden]; T <= max_tokens of the handle."""
        T = x.shape[0]
        y = torch.empty((T, self.hidden), dtype=torch.bfloat16, device=x.device)
        ids = wts = None
        if return_routing:
            ids = torch.empty((T, self.topk), dtype=torch.int16, device=x.device)
            wts = torch.empty((T, self.topk), dtype=torch.float32, device=x.device)
        _check(load().blok_moe_batched(self._handle, _ptr(x, torch.bfloat16, "x"), C.c_int(T), _ptr(y), _ptr(ids), _ptr(wts),
                                       _stream()))
        return (y, ids, wts) if return_routing else y

    def check(self):
        """Synchronises the stream and raises if a device-side bounded wait gave up (blok_moe_layer_check)."""
        _check(load().blok_moe_layer_check(self._handle, _stream()))

    def experts_grouped(self, x, expert_local, x_index=None):
        """y[a] = bf16(expert_{expert_local[a]}(x[x_index[a]])) for N assignments (the expert-parallel building block)."""
        N = expert_local.numel()
        y = torch.empty((N, self.hidden), dtype=torch.bfloat16, device=x.device)
        _check(load().blok_moe_experts_grouped(self._handle, _ptr(x, torch.bfloat16, "x"), _ptr(x_index, torch.int32),
                                               _ptr(expert_local, torch.int32, "expert_local"), C.c_int(N), _ptr(y),
                                               _stream()))
        return y

    def shared(self, x):
        """The shared expert for T tokens (bf16_mlp, src/kimi_exec.cu:872-875)."""
        T = x.shape[0]
        out = torch.empty((T, self.hidden), dtype=torch.bfloat16, device=x.device)
        _check(load().blok_moe_shared(self._handle, _ptr(x, torch.bfloat16, "x"), C.c_int(T), _ptr(out), _stream()))
        return out

    def decode_host(self, x_host, y_host):
        """Host-buffer call: x_host / y_host are (ideally pinned) CPU bf16 tensors of [hidden]; returns after the
        result has landed in y_host."""
        if x_host.is_cuda or y_host.is_cuda:
            raise BlokError(-1, "decode_host takes CPU tensors")
        if x_host.dtype != torch.bfloat16 or y_host.dtype != torch.bfloat16 or x_host.numel() != self.hidden or \
                y_host.numel() != self.hidden or not x_host.is_contiguous() or not y_host.is_contiguous():
            raise BlokError(-1, "decode_host needs contiguous bf16 [hidden] tensors")
        with torch.cuda.device(self.device):
            _check(load().blok_moe_decode_host(self._handle, C.c_void_p(x_host.data_ptr()), C.c_void_p(y_host.data_ptr()),
                                               _stream()))
        return y_host


def _moe_weights_struct(w, topk, routed_scale, expert_base):
    E, H = w["router_w"].shape
    n, I = w["gate_w"].shape[0], w["gate_w"].shape[1]
    S = w["shared_gate"].shape[0] if w.get("shared_gate") is not None else 0
    return MoeWeights(
        hidden=H, inter=I, experts=E, topk=topk, shared_inter=S, routed_scale=routed_scale,
        router_w=_ptr(w["router_w"], torch.bfloat16, "router_w").value,
        router_bias=_ptr(w["router_bias"], torch.float32, "router_bias").value,
        expert_base=expert_base, experts_local=n,
        gate_w=_ptr(w["gate_w"], torch.int32, "gate_w").value, gate_s=_ptr(w["gate_s"], torch.bfloat16, "gate_s").value,
        up_w=_ptr(w["up_w"], torch.int32, "up_w").value, up_s=_ptr(w["up_s"], torch.bfloat16, "up_s").value,
        down_w=_ptr(w["down_w"], torch.int32, "down_w").value, down_s=_ptr(w["down_s"], torch.bfloat16, "down_s").value,
        shared_gate=_ptr(w.get("shared_gate"), torch.bfloat16).value,
        shared_up=_ptr(w.get("shared_up"), torch.bfloat16).value,
        shared_down=_ptr(w.get("shared_down"), torch.bfloat16).value,
    )


COMM_ID_BYTES = 128


def comm_unique_id():
    """128 bytes that one rank creates and every rank passes to Comm (blok_comm_unique_id)."""
    buf = C.create_string_buffer(COMM_ID_BYTES)
    _check(load().blok_comm_unique_id(buf))
    return bytes(buf.raw)


class Comm:
    """The library's communicator (blok_comm_*): one per process, on the current CUDA device.  With `group` (or an
    initialised torch.distributed default group) rank 0 creates the id and broadcasts it over that group; the
    communicator itself is the library's own (NCCL resolved inside the library)."""

    def __init__(self, rank=None, world=None, unique_id=None, group=None):
        import torch.distributed as dist
        if rank is None:
            rank = dist.get_rank(group) if dist.is_initialized() else 0
            world = dist.get_world_size(group) if dist.is_initialized() else 1
        if world > 1 and unique_id is None:
            holder = [comm_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(holder, src=0, group=group)
            unique_id = holder[0]
        self.rank, self.world = rank, world
        self._handle = C.c_void_p()
        idbuf = C.create_string_buffer(unique_id, COMM_ID_BYTES) if unique_id is not None else None
        _check(load().blok_comm_create(idbuf, C.c_int(rank), C.c_int(world), C.byref(self._handle)))

    def close(self):
        if getattr(self, "_handle", None) is not None and self._handle.value:
            load().blok_comm_destroy(self._handle)
            self._handle = C.c_void_p()

    def check(self):
        _check(load().blok_comm_check(self._handle))

    def all_reduce_(self, t):
        """In-place sum over the ranks of a float32 CUDA tensor."""
        _check(load().blok_comm_all_reduce_f32(self._handle, _ptr(t, torch.float32), C.c_long(t.numel()), _stream()))
        return t

    def broadcast_(self, t, root=0):
        _check(load().blok_comm_broadcast(self._handle, _ptr(t), C.c_long(t.numel() * t.element_size()), C.c_int(root), _stream()))
        return t


class MoeEp:
    """The expert-parallel batched layer (blok_moe_ep_*).  `weights` as for MoeLayer, the expert arrays holding this
    rank's experts [experts / world, ...] only; router and shared expert replicated."""

    def __init__(self, comm, weights, topk=8, routed_scale=2.827, max_tokens=256):
        self.comm, self.weights = comm, dict(weights)
        E, H = weights["router_w"].shape
        per = E // comm.world
        self.hidden, self.topk, self.experts, self.max_tokens = H, topk, E, max_tokens
        mw = _moe_weights_struct(self.weights, topk, routed_scale, comm.rank * per)
        self._handle = C.c_void_p()
        self.device = weights["router_w"].device
        with torch.cuda.device(self.device):
            _check(load().blok_moe_ep_create(comm._handle, C.byref(mw), C.c_int(max_tokens), C.byref(self._handle)))

    def close(self):
        if getattr(self, "_handle", None) is not None and self._handle.value:
            load().blok_moe_ep_destroy(self._handle)
            self._handle = C.c_void_p()

    def forward(self, x, out=None, return_routing=False):
        """x bf16 [T, hidden] (this rank's tokens) -> y bf16 [T, hidden]; every rank calls it once per pass."""
        T = x.shape[0]
        y = torch.empty((T, self.hidden), dtype=torch.bfloat16, device=x.device) if out is None else out
        ids = wts = None
        if return_routing:
            ids = torch.empty((T, self.topk), dtype=torch.int16, device=x.device)
            wts = torch.empty((T, self.topk), dtype=torch.float32, device=x.device)
        _check(load().blok_moe_ep_forward(self._handle, _ptr(x, torch.bfloat16, "x"), C.c_int(T), _ptr(y, torch.bfloat16), _ptr(ids),
                                          _ptr(wts), _stream()))
        return (y, ids, wts) if return_routing else y

    def check(self):
        _check(load().blok_moe_ep_check(self._handle, _stream()))

    def profile(self, on=True):
        _check(load().blok_moe_ep_profile(self._handle, C.c_int(1 if on else 0)))

    def phase_ms(self):
        """Device milliseconds of the last pass by phase (profiling must be on); waits for the pass."""
        out = (C.c_float * 6)()
        _check(load().blok_moe_ep_phase_ms(self._handle, out))
        return dict(zip(("route", "dispatch", "shared", "wait_rows", "experts", "combine"), [float(v) for v in out]))

    def stats(self):
        """After a pass: assignments sent, of those to other ranks, rows received, GEMM tiles (synchronises)."""
        out = (C.c_longlong * 4)()
        _check(load().blok_moe_ep_stats(self._handle, out, _stream()))
        return dict(assignments=out[0], remote=out[1], received=out[2], tiles=out[3],
                    bytes_each_way=out[1] * self.hidden * 2)


def lm_head_argmax(w, n):
    """Greedy sampler (src/kimi_exec.cu:718-734): n bf16 [T<=64, hidden] -> token ids int32 [T] on the device."""
    vocab, hidden = w.shape
    n2 = n.reshape(-1, hidden)
    T = n2.shape[0]
    lib = load()
    lib.blok_lm_head_workspace_bytes.restype = C.c_size_t
    need = lib.blok_lm_head_workspace_bytes(C.c_int(vocab), C.c_int(T))
    ws = torch.empty(need, dtype=torch.uint8, device=n.device)
    ids = torch.empty(T, dtype=torch.int32, device=n.device)
    _check(lib.blok_lm_head_argmax(_ptr(w, torch.bfloat16), _ptr(n2, torch.bfloat16), C.c_int(vocab), C.c_int(hidden),
                                   C.c_int(T), _ptr(ids), _ptr(ws), C.c_size_t(need), _stream()))
    return ids


def embed(table, ids):
    """embed_token (src/kimi_exec.cu:651-655): ids int32 [T] on the device -> bf16 [T, hidden]."""
    vocab, hidden = table.shape
    x = torch.zeros((ids.numel(), hidden), dtype=torch.bfloat16, device=table.device)
    _check(load().blok_embed(_ptr(table, torch.bfloat16), _ptr(ids, torch.int32), C.c_int(vocab), C.c_int(hidden),
                             C.c_int(ids.numel()), _ptr(x), _stream()))
    return x


class MlaWeights(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("hidden", "heads", "qk_nope", "qk_rope", "v_head", "q_rank", "kv_rank")] + \
               [(n, C.c_float) for n in ("rms_eps", "rope_theta", "yarn_factor", "yarn_beta_fast", "yarn_beta_slow",
                                         "yarn_original_ctx", "yarn_mscale_all_dim")] + \
               [(n, C.c_void_p) for n in ("q_a", "q_a_ln", "q_b", "kv_a", "kv_a_ln", "kv_b", "o")]


class MlaLayer:
    """Handle of one MLA attention block (src/kimi_exec.cu:813-826 + :692-716) in the absorbed form over a bf16
    latent cache.  `weights`: dict of CUDA bf16 tensors q_a [1536,7168], q_a_ln [1536], q_b [12288,1536],
    kv_a [576,7168], kv_a_ln [512], kv_b [16384,512], o [7168,8192].  The tensors are borrowed."""

    def __init__(self, weights, yarn_factor=64.0, rope_theta=50000.0, rms_eps=1e-5, max_batch=8, max_ctx=32768,
                 heads=64, qk_nope=128, qk_rope=64, v_head=128):
        self.weights = dict(weights)
        w = self.weights
        q_rank, hidden = w["q_a"].shape
        kv_rank = w["kv_a_ln"].shape[0]
        self.hidden, self.heads, self.kv_rank, self.qk_rope = hidden, heads, kv_rank, qk_rope
        self.lat_w = kv_rank + qk_rope
        self._w = MlaWeights(hidden=hidden, heads=heads, qk_nope=qk_nope, qk_rope=qk_rope, v_head=v_head, q_rank=q_rank,
                             kv_rank=kv_rank, rms_eps=rms_eps, rope_theta=rope_theta, yarn_factor=yarn_factor,
                             yarn_beta_fast=32.0, yarn_beta_slow=1.0, yarn_original_ctx=4096.0, yarn_mscale_all_dim=1.0,
                             **{k: _ptr(w[k], torch.bfloat16, k).value for k in ("q_a", "q_a_ln", "q_b", "kv_a", "kv_a_ln",
                                                                                 "kv_b", "o")})
        lib = load()
        lib.blok_mla_softmax_scale.restype = C.c_float
        self.scale = float(lib.blok_mla_softmax_scale(C.byref(self._w)))
        self._handle = C.c_void_p()
        self.device = w["q_a"].device
        with torch.cuda.device(self.device):
            _check(lib.blok_mla_layer_create(C.byref(self._w), C.c_int(max_batch), C.c_int(max_ctx), C.byref(self._handle)))

    def close(self):
        if getattr(self, "_handle", None) is not None and self._handle.value:
            load().blok_mla_layer_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def decode(self, n, cache, ctx_len, out=None):
        """n bf16 [B, hidden]; cache bf16 [B, ctx_stride, 576] (row ctx_len[b] is written); ctx_len int32 [B] (device)."""
        B = n.shape[0]
        y = torch.empty((B, self.hidden), dtype=torch.bfloat16, device=n.device) if out is None else out
        _check(load().blok_mla_decode(self._handle, _ptr(n, torch.bfloat16, "n"), _ptr(cache, torch.bfloat16, "cache"),
                                      C.c_long(cache.shape[1]), _ptr(ctx_len, torch.int32, "ctx_len"), C.c_int(B),
                                      _ptr(y, torch.bfloat16, "out"), _stream()))
        return y

    def check(self):
        """Synchronises and raises if an earlier decode call had a position outside its sequence's cache rows."""
        _check(load().blok_mla_layer_check(self._handle, _stream()))

    def attend(self, q, cache, seq_len, scale=None, out=None):
        """The attention core: q bf16 [B, heads, 576], seq_len int32 [B] (device) -> o_lat bf16 [B, heads, 512]."""
        B = q.shape[0]
        o = torch.empty((B, self.heads, self.kv_rank), dtype=torch.bfloat16, device=q.device) if out is None else out
        _check(load().blok_mla_attend(self._handle, _ptr(q, torch.bfloat16, "q"), _ptr(cache, torch.bfloat16, "cache"),
                                      C.c_long(cache.shape[1]), _ptr(seq_len, torch.int32, "seq_len"), C.c_int(B),
                                      C.c_float(self.scale if scale is None else scale), _ptr(o, torch.bfloat16, "o_lat"),
                                      _stream()))
        return o

    def prefill(self, n, cache, first_pos, out=None):
        """A prefill chunk of one sequence: n bf16 [T, hidden] (consecutive tokens), cache bf16 [ctx_cap, 576] (rows
        first_pos .. first_pos+T-1 are written), first_pos int32 [1] (device)."""
        T = n.shape[0]
        y = torch.empty((T, self.hidden), dtype=torch.bfloat16, device=n.device) if out is None else out
        _check(load().blok_mla_prefill(self._handle, _ptr(n, torch.bfloat16, "n"), _ptr(cache, torch.bfloat16, "cache"),
                                       C.c_long(cache.shape[0]), _ptr(first_pos, torch.int32, "first_pos"), C.c_int(T),
                                       _ptr(y, torch.bfloat16, "out"), _stream()))
        return y

    def decode_paged(self, n, pool, block_table, ctx_len, slot_of=None, out=None):
        """decode() over a paged pool: pool bf16 [pages, page_rows, 576], block_table int32 [slots, table_stride]
        (device), slot_of int32 [B] (device) or None for slot b."""
        B = n.shape[0]
        y = torch.empty((B, self.hidden), dtype=torch.bfloat16, device=n.device) if out is None else out
        _check(load().blok_mla_decode_paged(
            self._handle, _ptr(n, torch.bfloat16, "n"), _ptr(pool, torch.bfloat16, "pool"),
            _ptr(block_table, torch.int32, "block_table"), _ptr(slot_of, torch.int32, "slot_of") if slot_of is not None else None,
            C.c_int(block_table.shape[1]), C.c_int(pool.shape[1]), _ptr(ctx_len, torch.int32, "ctx_len"), C.c_int(B),
            _ptr(y, torch.bfloat16, "out"), _stream()))
        return y

    def attend_paged(self, q, pool, block_table, seq_len, slot_of=None, scale=None, out=None):
        """attend() over a paged pool."""
        B = q.shape[0]
        o = torch.empty((B, self.heads, self.kv_rank), dtype=torch.bfloat16, device=q.device) if out is None else out
        _check(load().blok_mla_attend_paged(
            self._handle, _ptr(q, torch.bfloat16, "q"), _ptr(pool, torch.bfloat16, "pool"),
            _ptr(block_table, torch.int32, "block_table"), _ptr(slot_of, torch.int32, "slot_of") if slot_of is not None else None,
            C.c_int(block_table.shape[1]), C.c_int(pool.shape[1]), _ptr(seq_len, torch.int32, "seq_len"), C.c_int(B),
            C.c_float(self.scale if scale is None else scale), _ptr(o, torch.bfloat16, "o_lat"), _stream()))
        return o


class KvPages:
    """Host-side page bookkeeping of a paged latent cache (blok_kv_pages_*): no GPU needed except upload()."""

    def __init__(self, n_pages, page_rows, slots, table_stride):
        self.n_pages, self.page_rows, self.slots, self.table_stride = n_pages, page_rows, slots, table_stride
        self._handle = C.c_void_p()
        _check(load().blok_kv_pages_create(C.c_int(n_pages), C.c_int(page_rows), C.c_int(slots), C.c_int(table_stride),
                                           C.byref(self._handle)))

    def close(self):
        if getattr(self, "_handle", None) is not None and self._handle.value:
            load().blok_kv_pages_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def reserve(self, slot, n_rows):
        _check(load().blok_kv_pages_reserve(self._handle, C.c_int(slot), C.c_long(n_rows)))

    def release(self, slot):
        _check(load().blok_kv_pages_release(self._handle, C.c_int(slot)))

    def fork(self, src_slot, dst_slot, n_rows):
        _check(load().blok_kv_pages_fork(self._handle, C.c_int(src_slot), C.c_int(dst_slot), C.c_long(n_rows)))

    @property
    def free(self):
        return int(load().blok_kv_pages_free_count(self._handle))

    def rows(self, slot):
        f = load().blok_kv_pages_rows
        f.restype = C.c_long
        return int(f(self._handle, C.c_int(slot)))

    def table(self):
        """A copy of the host table as a numpy int32 array [slots, table_stride]."""
        import numpy as np
        f = load().blok_kv_pages_table
        f.restype = C.POINTER(C.c_int)
        ptr = f(self._handle)
        return np.ctypeslib.as_array(ptr, shape=(self.slots, self.table_stride)).copy()

    def upload(self, device_table):
        _check(load().blok_kv_pages_upload(self._handle, _ptr(device_table, torch.int32, "device_table"), _stream()))


class Batcher:
    """Host-side continuous-batching scheduler (blok_batcher_*): no GPU needed."""

    def __init__(self, slots, n_pages, page_rows, max_ctx):
        self.slots = slots
        self._handle = C.c_void_p()
        _check(load().blok_batcher_create(C.c_int(slots), C.c_int(n_pages), C.c_int(page_rows), C.c_int(max_ctx),
                                          C.byref(self._handle)))

    def close(self):
        if getattr(self, "_handle", None) is not None and self._handle.value:
            load().blok_batcher_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def submit(self, n_prompt, max_new):
        rid = C.c_int(-1)
        _check(load().blok_batcher_submit(self._handle, C.c_int(n_prompt), C.c_int(max_new), C.byref(rid)))
        return rid.value

    def plan(self):
        """-> (admitted [(slot, request)], decode slots)"""
        A = C.c_int * self.slots
        a_s, a_r, d_s, na, nd = A(), A(), A(), C.c_int(0), C.c_int(0)
        _check(load().blok_batcher_plan(self._handle, a_s, a_r, C.byref(na), d_s, C.byref(nd)))
        return [(a_s[i], a_r[i]) for i in range(na.value)], [d_s[i] for i in range(nd.value)]

    def token(self, slot, is_eos=False):
        """Reports a sampled token of the sequence in `slot`; True when the sequence ended."""
        fin = C.c_int(0)
        _check(load().blok_batcher_token(self._handle, C.c_int(slot), C.c_int(1 if is_eos else 0), C.byref(fin)))
        return bool(fin.value)

    @property
    def unfinished(self):
        return int(load().blok_batcher_unfinished(self._handle))

    @property
    def waiting(self):
        return int(load().blok_batcher_waiting(self._handle))

    @property
    def committed_pages(self):
        f = load().blok_batcher_committed_pages
        f.restype = C.c_long
        return int(f(self._handle))

    def emitted(self, request):
        return int(load().blok_batcher_emitted(self._handle, C.c_int(request)))


class ModelConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("layers", "first_dense", "hidden", "vocab", "dense_inter", "inter", "experts", "topk",
                                       "shared_inter")] + [("routed_scale", C.c_float)] + \
               [(n, C.c_int) for n in ("heads", "qk_nope", "qk_rope", "v_head", "q_rank", "kv_rank")] + \
               [(n, C.c_float) for n in ("rms_eps", "final_rms_eps", "rope_theta", "yarn_factor", "yarn_beta_fast",
                                         "yarn_beta_slow", "yarn_original_ctx", "yarn_mscale_all_dim")] + \
               [("max_batch", C.c_int), ("max_ctx", C.c_int), ("eos_id", C.c_uint32), ("prefill_chunk", C.c_int),
                ("kv_page_rows", C.c_int), ("kv_pages", C.c_int), ("ep_rank", C.c_int), ("ep_world", C.c_int)]


def index_validate(path, cfg):
    """Parses a runtime index and checks the forward contract for cfg (no GPU needed): (tensors, bytes) to load."""
    n, b = C.c_long(0), C.c_ulonglong(0)
    _check(load().blok_index_validate(str(path).encode(), C.byref(cfg), C.byref(n), C.byref(b)))
    return n.value, b.value


def default_model_config(**overrides):
    cfg = ModelConfig()
    load().blok_model_default_config(C.byref(cfg))
    for k, v in overrides.items():
        if not hasattr(cfg, k):
            raise BlokError(-1, "unknown model config field %r" % k)
        setattr(cfg, k, v)
    return cfg


_cudart = None


def _rt():
    global _cudart
    if _cudart is None:
        for name in ("libcudart.so.12", "libcudart.so"):
            try:
                _cudart = C.CDLL(name)
                break
            except OSError:
                continue
        if _cudart is None:
            raise BlokError(-100, "libcudart not found")
    return _cudart


class Model:
    """The whole decode model with seeded synthetic weights (generate(), src/kimi_exec.cu:780-893)."""

    def __init__(self, seed=4, **overrides):
        lib = load()
        self.cfg = ModelConfig()
        lib.blok_model_default_config(C.byref(self.cfg))
        for k, v in overrides.items():
            if not hasattr(self.cfg, k):
                raise BlokError(-1, "unknown model config field %r" % k)
            setattr(self.cfg, k, v)
        self._handle = C.c_void_p()
        _check(lib.blok_model_create_synthetic(C.byref(self.cfg), C.c_uint64(seed), C.byref(self._handle)))

    def close(self):
        if getattr(self, "_handle", None) is not None and self._handle.value:
            load().blok_model_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_comm(self, comm):
        """Expert parallelism: the communicator of a model created with ep_world > 1 (kept alive by this object)."""
        _check(load().blok_model_set_comm(self._handle, comm._handle))
        self._comm = comm

    def check(self):
        """Synchronises; raises if a layer's device-side wait gave up, a position left its cache or the communicator failed."""
        _check(load().blok_model_check(self._handle, _stream()))

    def hidden(self, rows):
        """The final-normed hidden states of the last step's first `rows` sequences (blok_model_hidden): a bf16
        [rows, hidden] tensor copied off the model's buffer after a synchronise."""
        ptr, cap = C.c_void_p(), C.c_int()
        _check(load().blok_model_hidden(self._handle, C.byref(ptr), C.byref(cap)))
        if rows > cap.value:
            raise BlokError(-2, "hidden(): %d rows asked, the buffer holds %d" % (rows, cap.value))
        torch.cuda.synchronize()
        out = torch.empty((rows, self.cfg.hidden), dtype=torch.bfloat16, device="cuda")
        rc = _rt().cudaMemcpy(C.c_void_p(out.data_ptr()), ptr, C.c_size_t(out.numel() * 2), C.c_int(3))
        if rc != 0:
            raise BlokError(-3, "cudaMemcpy D2D failed: %d" % rc)
        return out

    def tensor(self, layer, name, dtype, shape=None):
        """Host copy (numpy) of a weight tensor."""
        import numpy as np
        ptr, nbytes = C.c_void_p(), C.c_size_t()
        _check(load().blok_model_tensor(self._handle, C.c_int(layer), name.encode(), C.byref(ptr), C.byref(nbytes)))
        torch.cuda.synchronize()
        out = np.empty(nbytes.value // np.dtype(dtype).itemsize, dtype)
        rc = _rt().cudaMemcpy(out.ctypes.data_as(C.c_void_p), ptr, C.c_size_t(nbytes.value), C.c_int(2))
        if rc != 0:
            raise BlokError(-3, "cudaMemcpy D2H failed: %d" % rc)
        return out.reshape(shape) if shape is not None else out

    def write_tensor(self, layer, name, array):
        """Overwrite a weight tensor from a numpy array of the same byte size."""
        ptr, nbytes = C.c_void_p(), C.c_size_t()
        _check(load().blok_model_tensor(self._handle, C.c_int(layer), name.encode(), C.byref(ptr), C.byref(nbytes)))
        if array.nbytes != nbytes.value:
            raise BlokError(-2, "size mismatch for %s" % name)
        torch.cuda.synchronize()
        rc = _rt().cudaMemcpy(ptr, array.ctypes.data_as(C.c_void_p), C.c_size_t(nbytes.value), C.c_int(1))
        if rc != 0:
            raise BlokError(-3, "cudaMemcpy H2D failed: %d" % rc)

    def load_index(self, path):
        """Replace the weights by the checkpoint a runtime index describes (blok_model_load_index)."""
        _check(load().blok_model_load_index(self._handle, str(path).encode()))

    def reset(self):
        _check(load().blok_model_reset(self._handle))

    def step(self, ids):
        """ids int32 [B] on the device -> next ids int32 [B] on the device."""
        nxt = torch.empty_like(ids)
        _check(load().blok_model_step(self._handle, _ptr(ids, torch.int32, "ids"), C.c_int(ids.numel()), _ptr(nxt), _stream()))
        return nxt

    def prefill(self, ids):
        """The next tokens of sequence 0 in chunks (blok_model_prefill): ids int32 [n] on the device -> the greedy id
        after the last one, int32 [1] on the device.  The model needs prefill_chunk >= 1."""
        nxt = torch.empty(1, dtype=torch.int32, device=ids.device)
        _check(load().blok_model_prefill(self._handle, _ptr(ids, torch.int32, "ids"), C.c_int(ids.numel()), _ptr(nxt), _stream()))
        return nxt

    def step_slots(self, slots, ids):
        """A step of the sequences in the given slots (host list of distinct ints); ids int32 [B] on the device in the
        same order.  On a paged model any subset of the resident sequences may step."""
        B = len(slots)
        arr = (C.c_int * B)(*slots)
        nxt = torch.empty_like(ids)
        _check(load().blok_model_step_slots(self._handle, arr, C.c_int(B), _ptr(ids, torch.int32, "ids"), _ptr(nxt), _stream()))
        return nxt

    def prefill_slot(self, slot, ids):
        """prefill() for the sequence in `slot` of a paged model."""
        nxt = torch.empty(1, dtype=torch.int32, device=ids.device)
        _check(load().blok_model_prefill_slot(self._handle, C.c_int(slot), _ptr(ids, torch.int32, "ids"), C.c_int(ids.numel()),
                                              _ptr(nxt), _stream()))
        return nxt

    def release_slot(self, slot):
        _check(load().blok_model_slot_release(self._handle, C.c_int(slot), _stream()))

    def slot_length(self, slot):
        f = load().blok_model_slot_length
        f.restype = C.c_long
        return int(f(self._handle, C.c_int(slot)))

    @property
    def free_pages(self):
        return int(load().blok_model_free_pages(self._handle))

    def generate_many(self, prompts, max_new):
        """Greedy generation for several prompts at once on a paged model (blok_model_generate_many): a list of token
        lists in, a list of token lists out, in the same order."""
        import numpy as np
        flat = np.ascontiguousarray([t for p in prompts for t in p], np.uint32)
        offs = np.zeros(len(prompts) + 1, np.int32)
        offs[1:] = np.cumsum([len(p) for p in prompts])
        out = np.zeros(len(prompts) * max_new, np.uint32)
        n = np.zeros(len(prompts), np.int32)
        _check(load().blok_model_generate_many(self._handle, flat.ctypes.data_as(C.c_void_p), offs.ctypes.data_as(C.c_void_p),
                                               C.c_int(len(prompts)), C.c_int(max_new), out.ctypes.data_as(C.c_void_p),
                                               n.ctypes.data_as(C.c_void_p)))
        return [out[r * max_new:r * max_new + n[r]].tolist() for r in range(len(prompts))]

    def generate(self, prompt, max_new):
        """Greedy generation with host token lists, like the reference executor's command line."""
        import numpy as np
        p = np.ascontiguousarray(prompt, np.uint32)
        out = np.zeros(max_new, np.uint32)
        n = C.c_int(0)
        _check(load().blok_model_generate(self._handle, p.ctypes.data_as(C.c_void_p), C.c_int(p.size), C.c_int(max_new),
                                          out.ctypes.data_as(C.c_void_p), C.byref(n)))
        return out[:n.value].tolist()
