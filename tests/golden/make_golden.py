"""Generates tests/golden/dequant_golden.npz.

Raw blocks come from a fixed numpy seed; the expected values come from the
third-party `gguf` Python package (gguf.quants.dequantize), the GGML ground
truth whose block order the reference states it follows
(crates/dyninfer-checkpoint-gguf/src/q4.rs:34-42). Run from the repo root:

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import gguf  # noqa: E402
from gguf import quants  # noqa: E402

from dyninfer_b200 import synth  # noqa: E402

QT = {"gguf.q4_0": gguf.GGMLQuantizationType.Q4_0, "gguf.q4_1": gguf.GGMLQuantizationType.Q4_1,
      "gguf.q8_0": gguf.GGMLQuantizationType.Q8_0, "gguf.q6_k": gguf.GGMLQuantizationType.Q6_K,
      "gguf.q4_k": gguf.GGMLQuantizationType.Q4_K, "gguf.q5_k": gguf.GGMLQuantizationType.Q5_K,
      "gguf.iq4_xs": gguf.GGMLQuantizationType.IQ4_XS}


def main():
    out = {}
    for i, (enc, qt) in enumerate(QT.items()):
        rows, cols = 6, 512
        raw = synth.random_weight(enc, rows, cols, 1234 + i)["data"]
        # edge blocks: zero scale, extreme nibbles, negative scale, f16 subnormal scale
        bsz = {"gguf.q4_0": 18, "gguf.q4_1": 20, "gguf.q8_0": 34, "gguf.q6_k": 210, "gguf.q4_k": 144,
               "gguf.q5_k": 176, "gguf.iq4_xs": 136}[enc]
        blk = raw.reshape(-1, bsz).copy()
        doff = 208 if enc == "gguf.q6_k" else 0
        blk[0, doff:doff + 2] = 0
        blk[1, doff:doff + 2] = np.array([0x8400], np.uint16).view(np.uint8)   # -6.1e-5
        blk[2, doff:doff + 2] = np.array([0x0001], np.uint16).view(np.uint8)   # smallest subnormal
        # K-quants: the packed scales; IQ4_XS: scales_h, scales_l and the first index bytes
        qoff = {"gguf.q4_k": 4, "gguf.q5_k": 4}.get(enc, 2 if doff == 0 else 0)
        blk[3, qoff:qoff + 16] = 0xFF
        blk[4, qoff:qoff + 16] = 0x00
        raw = blk.reshape(-1)
        ref = quants.dequantize(raw.reshape(rows, -1), qt).astype(np.float32)
        out[enc + ":raw"] = raw
        out[enc + ":f32"] = ref.reshape(rows, cols)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "dequant_golden.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
