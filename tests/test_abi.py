"""The C-ABI library: it builds for sm_100a, loads without a GPU, exports every
symbol the header declares, and rejects bad arguments with error codes (no
compute call is made here)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from blok_b200 import build
    build.build()
    import blok_b200
    return blok_b200.load()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "blok_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(blok_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = declared_functions()
    assert len(names) >= 10
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, "declared in include/blok_b200.h but not exported: %s" % missing


def test_version_and_error_string(lib):
    assert lib.blok_abi_version() == 3
    lib.blok_last_error.restype = C.c_char_p
    rc = lib.blok_i4_dequant(None, None, None, 1, 32, None)
    assert rc == -1
    assert b"null pointer" in lib.blok_last_error()


def test_argument_validation_needs_no_gpu(lib):
    p = C.c_void_p(16)  # a non-null, aligned dummy; validation fails before any launch
    assert lib.blok_i4_gemv(p, p, p, p, 16, 33, None) == -2            # cols % 32
    assert lib.blok_bf16_gemv(p, p, p, None, 16, 64, 9, None) == -2    # T > 8
    assert lib.blok_bf16_gemv(p, p, p, p, 16, 64, 1, None) == -1       # both outputs given
    assert lib.blok_rmsnorm(p, p, p, 1, 0, C.c_float(1e-5), None) == -2
    assert lib.blok_router(p, p, p, 1, 2048, 64, 8, C.c_float(1.0), p, p, p, C.c_size_t(1 << 30), None) == -2
    assert lib.blok_router(p, p, p, 4, 384, 64, 8, C.c_float(1.0), p, p, p, C.c_size_t(8), None) == -6   # workspace
    assert lib.blok_expert_ffn(p, p, p, p, p, p, p, p, 7168, 2048, p, C.c_size_t(16), None) == -6
    assert lib.blok_expert_ffn(p, p, p, p, p, p, p, p, 7000, 2048, p, C.c_size_t(1 << 20), None) == -2
    out = C.c_void_p()
    assert lib.blok_moe_layer_create(None, 1, C.byref(out)) == -1
    assert lib.blok_moe_layer_destroy(None) == 0
    # expert parallelism: argument errors come before NCCL or a device is touched
    assert lib.blok_comm_unique_id(None) == -1
    assert lib.blok_comm_create(None, 2, 2, C.byref(out)) == -1        # rank outside the world
    assert lib.blok_comm_create(None, 0, 2, C.byref(out)) == -1        # more than one rank needs an id
    assert lib.blok_comm_destroy(None) == 0
    assert lib.blok_moe_ep_create(None, None, 8, C.byref(out)) == -1
    assert lib.blok_moe_ep_destroy(None) == 0
    # zero-sized work is a no-op, not an error
    assert lib.blok_i4_gemv(p, p, p, p, 0, 64, None) == 0
    assert lib.blok_add_bf16(p, p, C.c_long(0), None) == 0


def test_missing_library_is_loud(monkeypatch, tmp_path):
    import blok_b200.lib as L
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(L.BlokError):
        L.load()
