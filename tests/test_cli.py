"""The executor's command-line contract (src/kimi_exec.cu:532-544, :895-904): flags in pairs, unknown flags and bad
arguments exit 1 with a message on stderr; success prints one JSON line."""
import json
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "blok_b200", "blok-kimi-exec")


@pytest.fixture(scope="module")
def exe():
    from blok_b200 import build
    build.build()
    assert os.path.exists(EXE)
    return EXE


def run(exe, *args):
    return subprocess.run([exe, *args], capture_output=True, text=True, timeout=600)


def test_argument_errors_exit_1_with_message(exe):
    for args, msg in ((["--index", "x", "--prompt-tokens", "1,2"], "bad args"),
                      (["--index"], "usage:"),
                      (["--bogus", "1"], "unknown flag: --bogus"),
                      (["--index", "x", "--prompt-tokens", "1,a", "--tokens", "2"], "bad prompt token"),
                      (["--index", "x", "--prompt-tokens", "999999", "--tokens", "2"], "prompt token outside vocabulary"),
                      (["--index", "x", "--prompt-tokens", "1", "--tokens", "0"], "bad args"),
                      (["--index", "x", "--prompt-tokens", "1", "--tokens", "2", "--prefill-chunk", "8"],
                       "index: runtime index: cannot open x"),
                      (["--index", "x", "--prompt-tokens", "1", "--tokens", "2"], "index: runtime index: cannot open x")):
        p = run(exe, *args)
        assert p.returncode == 1 and msg in p.stderr and p.stdout == "", (args, p.stderr)


@pytest.mark.gpu
def test_synthetic_run_prints_one_json_line(exe):
    p = run(exe, "--index", "unused", "--prompt-tokens", "5,6,7", "--tokens", "4", "--synthetic-seed", "1", "--layers", "2",
            "--experts", "16", "--vocab", "4096")
    assert p.returncode == 0, p.stderr
    lines = p.stdout.strip().splitlines()
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["status"] == "ok" and 1 <= len(d["token_ids"]) <= 4 and all(0 <= t < 4096 for t in d["token_ids"])


@pytest.mark.gpu
def test_index_run_reproduces_the_model_the_checkpoint_was_written_from(exe, tmp_path):
    """A miniature checkpoint dumped from a seeded model, then run through --index: same tokens as the model itself."""
    import numpy as np
    import util
    from blok_b200 import lib
    cfg = dict(layers=2, first_dense=1, hidden=1024, vocab=2048, dense_inter=512, inter=256, experts=16, topk=8, shared_inter=256,
               q_rank=256, max_batch=1, max_ctx=32)
    model = lib.Model(seed=21, **cfg)
    for l in range(1, 2):  # a checkpoint stores the router's correction bias as bf16
        model.write_tensor(l, "router_bias", util.bf16_np_to_f32(util.f32_to_bf16_np(model.tensor(l, "router_bias", np.float32))))
    want = model.generate([5, 6, 7], 6)
    path = util.write_checkpoint(str(tmp_path), util.checkpoint_tensors(model.cfg, lambda l, n, dt, sh: model.tensor(l, n, dt, sh)))
    model.close()
    p = run(exe, "--index", path, "--prompt-tokens", "5,6,7", "--tokens", "6", "--layers", "2", "--experts", "16", "--vocab", "2048",
            "--hidden", "1024", "--dense-inter", "512", "--inter", "256", "--shared-inter", "256", "--q-rank", "256")
    assert p.returncode == 0, p.stderr
    assert json.loads(p.stdout)["token_ids"] == want
    # a checkpoint that lacks a tensor is refused before anything runs
    lines = [l for l in open(path).read().splitlines() if " norm " not in l]
    open(path, "w").write("\n".join(lines) + "\n")
    p = run(exe, "--index", path, "--prompt-tokens", "5", "--tokens", "1", "--layers", "2", "--experts", "16", "--vocab", "2048",
            "--hidden", "1024", "--dense-inter", "512", "--inter", "256", "--shared-inter", "256", "--q-rank", "256")
    assert p.returncode == 1 and "missing tensor -1:-1:resident:norm" in p.stderr
