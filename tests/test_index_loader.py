"""The runtime-index reader and the forward contract (runtime_index / validate_forward_contract,
src/kimi_exec.cu:559-581, :736-778) on a miniature checkpoint written by the test: the checks need no GPU."""
import numpy as np
import pytest

import util

TINY = dict(layers=2, first_dense=1, hidden=256, vocab=64, dense_inter=512, inter=256, experts=16, topk=8, shared_inter=256,
            heads=2, q_rank=64, kv_rank=64, max_batch=1, max_ctx=16)


def _random_get(rng):
    def get(layer, name, dtype, shape):
        if dtype == np.float32:
            return rng.standard_normal(shape).astype(np.float32)
        return rng.integers(0, np.iinfo(dtype).max, size=shape, dtype=dtype)
    return get


@pytest.fixture()
def tiny(tmp_path):
    from blok_b200 import lib
    cfg = lib.default_model_config(**TINY)
    tensors = util.checkpoint_tensors(cfg, _random_get(np.random.default_rng(5)))
    return lib, cfg, tensors, tmp_path


def test_index_validates_and_counts(tiny):
    lib, cfg, tensors, tmp = tiny
    path = util.write_checkpoint(str(tmp), tensors)
    n, nbytes = lib.index_validate(path, cfg)
    assert n == len(tensors) == 2 * 9 + 3 + 2 + 3 + 6 * 16 + 3
    assert nbytes == sum(np.asarray(t[7]).nbytes for t in tensors)


def _rewrite(path, fn):
    lines = open(path).read().splitlines()
    open(path, "w").write("\n".join(fn(lines)) + "\n")


@pytest.mark.parametrize("what,mutate,needle", [
    ("header", lambda L: ["blok-runtime-index-v0"] + L[1:], "bad header"),
    ("not a tensor line", lambda L: L[:3] + ["tokenizer x"] + L[3:], "not a tensor line"),
    ("missing field", lambda L: L[:2] + [" ".join(L[2].split()[:-1])] + L[3:], "incomplete"),
    ("whitespace in path", lambda L: L[:2] + [L[2] + " extra"] + L[3:], "trailing fields"),
    ("duplicate key", lambda L: L + [L[5]], "duplicate tensor key"),
    ("missing tensor", lambda L: [l for l in L if " lm_head " not in l], "missing tensor -1:-1:resident:lm_head"),
    ("wrong dtype", lambda L: [l.replace(" bf16 ", " f16 ") if " o_proj " in l else l for l in L], "the model needs bf16"),
    ("wrong shape", lambda L: [l.replace(" 16x256 ", " 256x16 ") if " gate " in l else l for l in L], "the model needs bf16 16x256"),
    ("unaligned extent", lambda L: L[:2] + [" ".join(p if i != 8 else str(int(p) + 1) for i, p in enumerate(L[2].split()))] + L[3:],
     "invalid extent"),
    ("layer outside the model", lambda L: L + [L[2].replace(" 0 -1 ", " 7 -1 ", 1)], "outside the model"),
])
def test_index_contract_violations_name_the_problem(tiny, what, mutate, needle):
    lib, cfg, tensors, tmp = tiny
    path = util.write_checkpoint(str(tmp), tensors)
    _rewrite(path, mutate)
    with pytest.raises(lib.BlokError) as e:
        lib.index_validate(path, cfg)
    assert needle in str(e.value), (what, str(e.value))


def test_missing_index_file(tiny):
    lib, cfg, _, tmp = tiny
    with pytest.raises(lib.BlokError) as e:
        lib.index_validate(str(tmp / "nope.blok"), cfg)
    assert "cannot open" in str(e.value)
