"""Golden fixtures for the GGUF-layout oracle, generated with the third-party `gguf` package.

For each of the five block formats that package implements (Q4_0, Q8_0, Q4_K, Q6_K, MXFP4),
draw 64 seeded random blocks (rocmforge_b200.synth laws) plus a few blocks with extreme
header bytes, dequantise them with gguf.quants.dequantize, and store input bytes and fp32
output in gguf_fixtures.npz. `gguf` is not part of ROCmForge; it is an independent check
of the layout restatement in oracle/oracle.c.

Run:  python tests/golden/make_gguf_fixtures.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import gguf  # noqa: E402
from gguf import quants  # noqa: E402

from rocmforge_b200 import synth  # noqa: E402

TYPES = {synth.Q4_0: gguf.GGMLQuantizationType.Q4_0, synth.Q8_0: gguf.GGMLQuantizationType.Q8_0,
         synth.Q4_K: gguf.GGMLQuantizationType.Q4_K, synth.Q6_K: gguf.GGMLQuantizationType.Q6_K,
         synth.MXFP4: gguf.GGMLQuantizationType.MXFP4}


def main():
    out = {"gguf_version": np.array(getattr(gguf, "__version__", "0.19.0"))}
    for qt, gt in TYPES.items():
        rng = synth.rng_for(7000 + qt)
        bb, be = synth.block_bytes(qt, synth.GGUF), synth.block_elems(qt)
        blocks = synth.gen_packed(qt, synth.GGUF, 64 * be, rng).reshape(64, bb).copy()
        extra = rng.integers(0, 256, size=(8, bb), dtype=np.uint8)   # fully random headers (subnormal d, big exps)
        if qt == synth.MXFP4:
            extra[:, 0] = [0, 1, 2, 126, 127, 128, 200, 254]
        blocks = np.concatenate([blocks, extra], axis=0)
        ref = quants.dequantize(blocks, gt).astype(np.float32).reshape(-1)
        out[f"in_{synth.QNAMES[qt]}"] = blocks.reshape(-1)
        out[f"out_{synth.QNAMES[qt]}"] = ref
    np.savez_compressed(os.path.join(HERE, "gguf_fixtures.npz"), **out)
    print("wrote gguf_fixtures.npz")


if __name__ == "__main__":
    main()
