"""Generates tests/golden/dequant_witness.npz.

Independent witness for the dequantisers: the gguf-py package (0.19.0, third party) run
on seeded random blocks.  Its Q8_0, Q4_K and Q6_K decoders produce the same element
order as boostr's CPU kernels.  Its Q4_0 decoder does not: ggml puts the 16 low nibbles
first and the 16 high nibbles second, boostr interleaves them
(out[2i] = low nibble of byte i, out[2i+1] = high nibble;
src/quant/cpu/kernels/dequant_simple.rs:24-31), so the Q4_0 witness is gguf-py's output
re-ordered by that rule.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", ".."))

from gguf import GGMLQuantizationType as T  # noqa: E402
from gguf import quants  # noqa: E402

from boostr_b200 import synth  # noqa: E402
from boostr_b200.format import QuantFormat as F  # noqa: E402


def main() -> None:
    out = {}
    rng = synth.rng_for(15, 7)
    for fmt, t, nblk in [(F.Q4_0, T.Q4_0, 24), (F.Q8_0, T.Q8_0, 24), (F.Q4_K, T.Q4_K, 6), (F.Q6_K, T.Q6_K, 6)]:
        blocks = synth._GEN[fmt](rng, nblk)
        # widen the value range beyond the benchmark distribution: random fp16 scales of both signs
        b2 = blocks.reshape(nblk, fmt.block_bytes).copy()
        d = (rng.standard_normal(nblk).astype(np.float32) * 3.0).astype(np.float16).view(np.uint8).reshape(nblk, 2)
        off = {F.Q4_0: 0, F.Q8_0: 0, F.Q4_K: 0, F.Q6_K: 208}[fmt]
        b2[nblk // 2:, off:off + 2] = d[nblk // 2:]
        blocks = b2.reshape(-1)
        vals = quants.dequantize(blocks.reshape(nblk, -1), t).astype(np.float32).reshape(nblk, -1)
        if fmt is F.Q4_0:
            inter = np.empty_like(vals)
            inter[:, 0::2] = vals[:, :16]
            inter[:, 1::2] = vals[:, 16:]
            vals = inter
        out[f"{fmt.name}_blocks"] = blocks
        out[f"{fmt.name}_f32"] = vals.reshape(-1)
    path = os.path.join(os.path.dirname(__file__), "dequant_witness.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
