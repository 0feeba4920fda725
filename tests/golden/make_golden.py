"""Regenerates tests/golden/*.npz.  Run in a checkout that has the lex-gpu tree beside it:

    python tests/golden/make_golden.py /path/to/lex-gpu

decode_tables.npz comes from the reference's own Python statement of the two formats
(scripts/qwen_nvfp4.py:27-42, imported, not copied): E2M1[16] and E4M3[256] as float32, plus the
dequantised f32 weights of a small seeded matrix formed with those tables in that script's order
(`E2M1[nib] * scale`, then `* gs`, scripts/qwen_nvfp4.py:88-92).  The oracle is checked against them.

config0.npz holds this repository's oracle outputs for the README's CPU-interpreter example (m = n = 128, k = 64, seeded
inputs of lex_gpu_b200/inputs.py): y and the f16 bit patterns of the staged weights.  The reference keeps
no stored outputs for gemm_fp4, so this one is a regression pin of the oracle, not a reference vector.
"""
import importlib.util
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))


def main(ref_root: str) -> None:
    spec = importlib.util.spec_from_file_location("qwen_nvfp4", Path(ref_root) / "scripts" / "qwen_nvfp4.py")
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    from lex_gpu_b200 import inputs
    from oracle import oracle as O

    wq, ws, _ = inputs.make_weights(32, 128, seed_base=123)
    ws = ws.copy()
    ws[0, :8] = [0x00, 0x01, 0x07, 0x08, 0x7E, 0x80, 0x81, 0xFE]          # zero, subnormals, max, negatives
    gs = np.float32(0.8125)
    words = wq.view("<u4")
    nib = np.empty((32, 128), dtype=np.uint8)
    for kk in range(8):                                                    # scripts/qwen_nvfp4.py:79-82
        nib[:, kk::8] = (words >> (4 * kk)) & 0xF
    w = ref.E2M1[nib].reshape(32, -1)
    w = w * np.repeat(ref.E4M3[ws], 16, axis=1)
    w = (w * gs).astype(np.float32)
    np.savez_compressed(HERE / "decode_tables.npz", e2m1=ref.E2M1.astype(np.float32), e4m3=ref.E4M3.astype(np.float32),
                        wq=wq, ws=ws, gs=gs, w_f32=w)

    x, wq0, ws0, wg0 = inputs.make_case(128, 128, 64)
    np.savez_compressed(HERE / "config0.npz", y=O.gemm_fp4(x, wq0, ws0, wg0), w16=O.dequant_fp4_f16(wq0, ws0, wg0))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of alpibrusl/lex-gpu>")
    main(sys.argv[1])
