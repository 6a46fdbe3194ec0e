#!/usr/bin/env python3
"""Collect the reference's committed decoder goldens into one small fixture.

Run once, in a checkout that has the reference tree mounted:

    python tests/golden/make_golden.py /path/to/jitllm

It reads, as DATA, the known-answer files the reference's own tests assert
bit-exactness against:

  testdata/golden/dequant/q4_k_tiny.{in,f32}      llama.cpp dequantize_row_q4_K
  testdata/golden/dequant/q8_0_{gemma,minilm,stories}.{in,f32}
  testdata/golden/dequant/{q4_0_gemma,q4_0_stories,q5_k_tiny,q6_k_tiny}.{in,f32}
  format/quant/testdata/mxfp4.json                gguf-py MXFP4.dequantize_blocks

and writes tests/golden/ref_decoder_vectors.npz (raw block bytes + expected f32
bit patterns). The tests load only the .npz; the reference tree is not needed
at test time.
"""
import json
import os
import sys

import numpy as np


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path of the jitllm checkout>")
    ref = sys.argv[1]
    out = {}
    dq = os.path.join(ref, "testdata", "golden", "dequant")
    for name in ("q4_k_tiny", "q8_0_gemma", "q8_0_minilm", "q8_0_stories", "q4_0_gemma", "q4_0_stories", "q5_k_tiny",
                 "q6_k_tiny"):
        out[name + "_blocks"] = np.fromfile(os.path.join(dq, name + ".in"), dtype=np.uint8)
        out[name + "_bits"] = np.fromfile(os.path.join(dq, name + ".f32"), dtype="<u4")
    with open(os.path.join(ref, "format", "quant", "testdata", "mxfp4.json")) as f:
        g = json.load(f)
    out["mxfp4_blocks"] = np.frombuffer(bytes.fromhex(g["blocks"]), dtype=np.uint8)
    out["mxfp4_bits"] = np.asarray(g["bits"], dtype="<u4")
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_decoder_vectors.npz")
    np.savez_compressed(dst, **out)
    for k, v in out.items():
        print(f"{k}: {v.dtype} x {v.size}")
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main()
