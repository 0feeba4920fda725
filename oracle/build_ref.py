"""Compiles the reference's own CUDA kernels for this path, from its sources where they lie, for sm_100a.

TEST INFRASTRUCTURE ONLY (the checker and the on-box bar); nothing under lex_gpu_b200/ loads what this builds.

    python oracle/build_ref.py [--reference /path/to/lex-gpu] [--force]

Two kernels of lex-gpu can be built without its Rust toolchain, because their CUDA text is in the tree:

* the emitted decode matvec `matvec_nvfp4_17408x5120` - a complete translation unit kept as a golden file
  (crates/lex-msl/tests/golden/matvec_nvfp4_17408x5120_cuda.cu: f32 x, weights as f32, 2176 blocks of 256
  threads).  It is compiled unchanged; only a host launcher is appended.
* the hand-scheduled GEMM the model ships (crates/lex-msl/src/gemm.rs:89-320).  It exists as a Rust
  `format!` template whose placeholders and brace escapes read the same in Python's str.format.  This script
  reads the template and the snippet literals out of gemm.rs, applies the schedule rules of gemm.rs:111-139
  (tile sizes by token count, 2 x 4 or 2 x 2 warps, 16-byte loads) for the listed shapes, and takes the
  dialect's preamble (crates/lex-msl/src/dialect.rs:681-700, 768-791) from the golden file above, which is
  that preamble as emitted.  Nothing of the kernel text is kept in this repository: the instances are
  written under oracle/_ref/ (git-ignored) and compiled there, one shared object per kernel, each with an
  appended `lexref_launch` and `lexref_info`.

Without the reference tree (a GPU box) the script changes nothing and the prebuilt objects are used.
"""
from __future__ import annotations

import argparse
import os
import re
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
GOLDEN_MATVEC = "crates/lex-msl/tests/golden/matvec_nvfp4_17408x5120_cuda.cu"
GEMM_RS = "crates/lex-msl/src/gemm.rs"

# (m, n, k, residual) instances of the hand-scheduled GEMM, all with f16 activations (`_xh`): the headline
# shapes, and small and ragged-m cases in the spirit of crates/lex-cuda/tests/device_gpu.rs:210-305 with n
# a multiple of 128 so that both implementations take them.
GEMM_INSTANCES = [
    (512, 17408, 5120, False),
    (512, 5120, 17408, True),
    (256, 512, 1024, False),
    (96, 256, 1024, True),
    (17, 128, 256, False),
    (40, 128, 512, False),
]


def reference_root(arg: str | None) -> Path | None:
    for cand in (arg, os.environ.get("LEX_REFERENCE"), "/root/reference"):
        if cand and (Path(cand) / GEMM_RS).exists():
            return Path(cand)
    return None


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def compile_so(cu: Path, so: Path) -> None:
    cmd = [nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
           "-Xcompiler", "-fPIC", "-w", "-o", str(so), str(cu)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"nvcc failed on {cu}")


def launcher(entry: str, params: list[str], gx: int, gy: int, threads: int) -> str:
    """Host code appended to a kernel: launch on a given stream with positional device pointers."""
    args = ", ".join(f"({ty})bufs[{i}]" for i, ty in enumerate(params))
    return f"""

// ---- appended by oracle/build_ref.py: host launcher (not part of the reference's text)
extern "C" __attribute__((visibility("default"))) int lexref_launch(void* const* bufs, int nbufs, void* stream)
{{
    if (nbufs != {len(params)}) return -1;
    {entry}<<<dim3({gx}u, {gy}u, 1u), dim3({threads}u, 1u, 1u), 0, (cudaStream_t)stream>>>({args});
    return (int)cudaGetLastError();
}}
extern "C" __attribute__((visibility("default"))) const char* lexref_info(void)
{{
    return "{entry} grid {gx}x{gy} threads {threads}";
}}
"""


# ---------------------------------------------------------------- reading Rust string literals

def rust_unescape(body: str) -> str:
    """The value of an ordinary Rust string literal's body: \\n, \\xNN, \\", \\\\ and the line continuation
    (a backslash before a newline swallows the newline and the next line's leading white space)."""
    out, i = [], 0
    while i < len(body):
        c = body[i]
        if c != "\\":
            out.append(c)
            i += 1
            continue
        nxt = body[i + 1]
        if nxt == "n":
            out.append("\n")
            i += 2
        elif nxt == "x":
            out.append(chr(int(body[i + 2:i + 4], 16)))
            i += 4
        elif nxt in "\"\\'":
            out.append(nxt)
            i += 2
        elif nxt == "t":
            out.append("\t")
            i += 2
        elif nxt == "\n":
            i += 2
            while i < len(body) and body[i] in " \t\n":
                i += 1
        else:
            raise ValueError(f"escape \\{nxt} not handled")
    return "".join(out)


def string_literals(src: str) -> list[str]:
    """Every string literal of a Rust source, raw (r#"..."#) or ordinary, as its value, in order.  Line
    comments outside literals are skipped (they may hold quotes); text inside a literal is kept as it is."""
    vals, i, n = [], 0, len(src)
    while i < n:
        if src.startswith("//", i):
            j = src.find("\n", i)
            i = n if j < 0 else j + 1
        elif src.startswith('r#"', i):
            j = src.index('"#', i + 3)
            vals.append(src[i + 3:j])
            i = j + 2
        elif src[i] == '"':
            j = i + 1
            while src[j] != '"':
                j += 2 if src[j] == "\\" else 1
            vals.append(rust_unescape(src[i + 1:j]))
            i = j + 1
        elif src[i] == "'":
            mt = re.compile(r"'(\\.|[^\\'])'").match(src, i)       # a char literal; else a lifetime tick
            i = mt.end() if mt else i + 1
        else:
            i += 1
    return vals


def literal(lits: list[str], starts: str) -> str:
    hits = [v for v in lits if v.startswith(starts)]
    if len(hits) != 1:
        raise RuntimeError(f"expected one literal starting {starts!r} in gemm.rs, found {len(hits)}")
    return hits[0]


def gemm_source(root: Path, preamble_includes: str, preamble_fp4: str, m: int, n: int, k: int, residual: bool):
    """One instance of gemm.rs's CUDA kernel with f16 activations, and its launch shape."""
    text = (root / GEMM_RS).read_text()
    start = text.index("fn cuda(")
    end = text.index("fn metal(")
    lits = string_literals(text[start:end])
    template = literal(lits, "// Generated by lex-msl::gemm.")
    aload_t = literal(lits, "for (uint e = tid; e < {bm}u * {bk}u / 8u;")
    eight = literal(lits, "*reinterpret_cast<const uint4*>(&x[(m0 + rr) * K + k0 + c])")
    bstore = literal(lits, "__half2 h[8];")
    rparam = literal(lits, "    const float* __restrict__ r,")
    radd_t = literal(lits, " + r[(row + rr) * N + col + c]")
    rfrag = literal(lits, "wmma::fragment<wmma::accumulator, 16, 16, 16, float> rf;")
    # schedule, gemm.rs:111-139 with no LEX_GEMM_CU_* override
    full = m > 64
    bm = 32 if m <= 32 else (128 if full else 64)
    bn = 128 if full else 64
    bk = 64 if (full and k % 64 == 0) else 32
    wgm, wgn = 2, (4 if full else 2)
    threads = 32 * wgm * wgn
    wtm, wtn = bm // wgm, bn // wgn
    fm, fnn = wtm // 16, wtn // 16
    bkp = bk + 8
    entry = f"gemm_nvfp4_{m}x{n}x{k}{'_res' if residual else ''}_xh"
    aload = aload_t.format(bm=bm, bk=bk, threads=threads, eight=eight)
    gx, gy = -(-n // bn), -(-m // bm)
    src = template.format(
        entry=entry, gx=gx, gy=gy, threads=threads, includes=preamble_includes, fp4=preamble_fp4, pack8="",
        xt="__half", rparam=rparam if residual else "", m=m, n=n, k=k, bn=bn, bm=bm, wgn=wgn, bkp=bkp,
        warps=wgm * wgn, fm=fm, fnn=fnn, bk=bk, aload=aload, bstore=bstore, wtm=wtm, wtn=wtn,
        rfrag=rfrag if residual else "", radd_t=radd_t if residual else "")
    params = ["const __half*", "const char*", "const char*", "const float*"] + (["const float*"] if residual else []) + ["float*"]
    return entry, src, params, gx, gy, threads


def build(reference: str | None = None, force: bool = False) -> list[Path]:
    root = reference_root(reference)
    if root is None:
        return sorted(OUT.glob("*.so"))        # a box without the reference tree: what was built earlier
    OUT.mkdir(exist_ok=True)
    built = []
    golden = (root / GOLDEN_MATVEC).read_text()
    newest_src = max((root / GOLDEN_MATVEC).stat().st_mtime, (root / GEMM_RS).stat().st_mtime, Path(__file__).stat().st_mtime)

    def fresh(so: Path) -> bool:
        return not force and so.exists() and so.stat().st_mtime >= newest_src

    # 1. the emitted matvec, unchanged, plus a launcher
    so = OUT / "matvec_nvfp4_17408x5120.so"
    if not fresh(so):
        cu = OUT / "matvec_nvfp4_17408x5120.cu"
        cu.write_text(golden + launcher("matvec_nvfp4_17408x5120",
                                        ["const float*", "const char*", "const char*", "const float*", "float*"],
                                        2176, 1, 256))
        compile_so(cu, so)
    built.append(so)

    # 2. the hand-scheduled GEMM, instantiated from gemm.rs's own template
    first_include = golden.index("#include <cuda_fp16.h>")
    tables = golden.index("__constant__ float FP4_V[16]")
    kernel = golden.index('extern "C" __global__')
    includes = "\n" + golden[first_include:tables]               # Cuda::includes()
    fp4 = golden[tables:kernel].rstrip("\n") + "\n"              # Cuda::fp4_preamble()
    for m, n, k, residual in GEMM_INSTANCES:
        entry, src, params, gx, gy, threads = gemm_source(root, includes, fp4, m, n, k, residual)
        so = OUT / f"{entry}.so"
        if not fresh(so):
            cu = OUT / f"{entry}.cu"
            cu.write_text(src + launcher(entry, params, gx, gy, threads))
            compile_so(cu, so)
        built.append(so)
    return built


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    for p in build(a.reference, a.force):
        print(p)
