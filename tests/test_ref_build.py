"""The recipe that compiles the reference's own CUDA kernels (oracle/build_ref.py): its reader of Rust string
literals, and - where the objects have been built - that each exports the appended launcher."""
import ctypes

import pytest

from oracle import build_ref, refkernels as R


def test_rust_literals_are_read_as_the_compiler_reads_them():
    src = r'''
        // a comment with a "quote" in it
        let a = "line one\n\
                 \x20   indented {x}u";
        let b = r#"raw {{ braces }} and "quotes" {y}"#;   // trailing "comment"
        let c = 'c'; let d: &'static str = "after a lifetime";
    '''
    lits = build_ref.string_literals(src)
    assert lits == ["line one\n    indented {x}u", 'raw {{ braces }} and "quotes" {y}', "after a lifetime"]
    assert lits[0].format(x=7) == "line one\n    indented 7u"
    assert lits[1].format(y=1) == 'raw { braces } and "quotes" 1'


def test_schedule_follows_the_token_count():
    """gemm.rs:111-139: 128 x 128 tiles, K steps of 64 and 8 warps above 64 tokens; 64-wide tiles with 4 warps
    at or below, 32 tokens tall at or below 32."""
    root = build_ref.reference_root(None)
    if root is None:
        pytest.skip("the reference tree is not on this machine")
    entry, src, params, gx, gy, threads = build_ref.gemm_source(root, "", "", 512, 17408, 5120, False)
    assert (entry, gx, gy, threads, len(params)) == ("gemm_nvfp4_512x17408x5120_xh", 136, 4, 256, 5)
    assert "__half As[128][72]" in src and "{" + "bm}" not in src
    entry, src, params, gx, gy, threads = build_ref.gemm_source(root, "", "", 17, 128, 256, True)
    assert (entry, gx, gy, threads, len(params)) == ("gemm_nvfp4_17x128x256_res_xh", 2, 1, 128, 6)
    assert "__half As[32][40]" in src and "const float* __restrict__ r," in src


def test_built_objects_export_the_launcher():
    entries = R.built_entries()
    if not entries:
        pytest.skip("oracle/_ref holds no built kernels on this machine")
    assert R.MATVEC_ENTRY in entries and R.gemm_entry(512, 17408, 5120) in entries
    for e in entries:
        lib = ctypes.CDLL(str(R.REF / f"{e}.so"))
        assert hasattr(lib, "lexref_launch") and hasattr(lib, "lexref_info")
        assert R.info(e).startswith(e)
