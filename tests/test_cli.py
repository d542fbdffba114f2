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
                      (["--index", "x", "--prompt-tokens", "1", "--tokens", "2"], "runtime index is not built")):
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
