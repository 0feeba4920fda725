"""bench.py's command line (no GPU): the option that times other token counts is for single-kernel runs only,
so the default run and the reference arm always measure the metric's own m = 512."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_tokens_needs_the_single_kernel_run():
    r = run("--tokens", "256")
    assert r.returncode == 2 and "--tokens is for --only gemm" in r.stderr
    r = run("--tokens", "256", "--only", "matvec")
    assert r.returncode == 2
    r = run("--tokens", "256", "--only", "gemm", "--impl", "reference")
    assert r.returncode == 2


def test_help_lists_the_contract_flags():
    r = run("--help")
    assert r.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--only", "--tokens", "--no-sustained"):
        assert flag in r.stdout
