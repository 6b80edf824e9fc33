"""Writes tests/golden/golden.npz: outputs of the CPU oracle on the reference's own in-code generators.

The reference holds no binary golden files for this path; its tests generate packed blocks and inputs in code
(`packed_blocks`, src/kernel/cpu/ggml_quant.rs:370-414; input formula `((i*17 % 101) - 50) / 64`, :432).  This script
restates those generators (tests/helpers.py), runs the oracle on them and stores bytes, dequantised values and
layer outputs, so that (a) a later change of the oracle shows up as a diff against committed numbers and (b) the GPU
tests have fixed vectors that do not depend on the oracle being rebuilt.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle as orc  # noqa: E402
from tests import helpers as H  # noqa: E402

TYPES = {"q4_0": 2, "q8_0": 8, "q4_k": 12, "iq4_nl": 20}
ROWS, COLS, TOKENS = 24, 512, 3


def inputs(tokens: int, cols: int) -> np.ndarray:
    i = np.arange(tokens * cols, dtype=np.int64)
    return (((i * 17 % 101).astype(np.float32) - 50.0) / 64.0).reshape(tokens, cols)


def main() -> None:
    out = {}
    x = inputs(TOKENS, COLS)
    out["x"] = x
    for name, t in TYPES.items():
        block = 256 if t == 12 else 32
        # types 8 and 12: the reference's generator (one "row" of it = 256 weights); 2 and 20: seeded
        # N(0, 0.02) weights through the round-to-nearest test encoders (the reference has no generator for them)
        packed = H.reference_packed_blocks(t, ROWS * COLS // 256) if t in (8, 12) else H.random_weight(t, ROWS, COLS, seed=2024 + t)
        out[f"{name}_bytes"] = packed
        out[f"{name}_dequant"] = orc.dequantize(t, packed, ROWS * COLS)
        out[f"{name}_matvec"] = orc.matvec(t, packed, ROWS, COLS, x[0])
        out[f"{name}_matmul"] = orc.matmul(t, packed, ROWS, COLS, x)
        half = ROWS // 2 * (COLS // block) * (len(packed) // (ROWS * COLS // block))
        out[f"{name}_gated"] = orc.gated_silu_matvec(t, packed[:half], packed[half:], ROWS // 2, COLS, x[0])
    values = (np.sin(np.arange(4 * 256, dtype=np.float32) * 0.37) * 0.05).astype(np.float32)
    out["q4_k_encode_in"] = values
    out["q4_k_encode_bytes"] = orc.encode_q4_k(values)
    logits = inputs(4, 16) * 3.0
    ids, w = orc.route_softmax_logits(logits, 4, 1.5, True)
    out["route_logits"], out["route_ids"], out["route_weights"] = logits, ids, w
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
