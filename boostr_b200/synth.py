"""Seeded synthetic inputs for the quantized-linear path.

The benchmark configurations describe their inputs as distributions, not data sets:
block scales are |N(0,1)| times a constant stored as fp16, quantised codes are uniform
over their range, activations are N(0,1).  These generators draw exactly that, on the
host with numpy's PCG64, so the same bytes can be handed to the CUDA library and to the
CPU checker.  Scale/min packing for Q4_K inverts the 6-bit unpack of
``unpack_q4k_q5k_scales`` (src/quant/cpu/kernels/dequant_k_quants/q4k_q5k.rs:108-122).
"""
from __future__ import annotations

import numpy as np

from .format import QuantFormat

SEED_BASE = 0xB2000000


def rng_for(config: int, tensor_index: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(SEED_BASE + 16 * config + tensor_index))


def activations(rng: np.random.Generator, m: int, k: int) -> np.ndarray:
    return rng.standard_normal((m, k), dtype=np.float32)


def _fp16_scale_bytes(rng: np.random.Generator, nblocks: int, mult: float) -> np.ndarray:
    d = (np.abs(rng.standard_normal(nblocks, dtype=np.float32)) * np.float32(mult)).astype(np.float16)
    return d.view(np.uint8).reshape(nblocks, 2)


def q4_0_blocks(rng, nblocks: int, scale: float = 0.02) -> np.ndarray:
    out = np.empty((nblocks, 18), dtype=np.uint8)
    out[:, 0:2] = _fp16_scale_bytes(rng, nblocks, scale)
    out[:, 2:18] = rng.integers(0, 256, size=(nblocks, 16), dtype=np.uint8)
    return out.reshape(-1)


def q8_0_blocks(rng, nblocks: int, scale: float = 0.004) -> np.ndarray:
    out = np.empty((nblocks, 34), dtype=np.uint8)
    out[:, 0:2] = _fp16_scale_bytes(rng, nblocks, scale)
    out[:, 2:34] = rng.integers(-127, 128, size=(nblocks, 32), dtype=np.int8).view(np.uint8)
    return out.reshape(-1)


def q5_0_blocks(rng, nblocks: int, scale: float = 0.01) -> np.ndarray:
    """Q5_0: f16 d, 32 high bits, 16 bytes of nibbles, all uniform, so the 5-bit codes are uniform 0..31."""
    out = np.empty((nblocks, 22), dtype=np.uint8)
    out[:, 0:2] = _fp16_scale_bytes(rng, nblocks, scale)
    out[:, 2:22] = rng.integers(0, 256, size=(nblocks, 20), dtype=np.uint8)
    return out.reshape(-1)


def q2_k_blocks(rng, nblocks: int, scale: float = 0.01) -> np.ndarray:
    """Q2_K: 16 scale bytes (4-bit scale, 4-bit min), 64 bytes of 2-bit codes, f16 d, f16 dmin; all fields uniform."""
    out = np.empty((nblocks, 84), dtype=np.uint8)
    out[:, 0:80] = rng.integers(0, 256, size=(nblocks, 80), dtype=np.uint8)
    out[:, 80:82] = _fp16_scale_bytes(rng, nblocks, scale)
    out[:, 82:84] = _fp16_scale_bytes(rng, nblocks, scale)
    return out.reshape(-1)


def q3_k_blocks(rng, nblocks: int, scale: float = 0.002) -> np.ndarray:
    """Q3_K: 32 B high-bit masks, 64 B of 2-bit codes, 12 B packed 6-bit scales, f16 d; all fields uniform."""
    out = np.empty((nblocks, 110), dtype=np.uint8)
    out[:, 0:108] = rng.integers(0, 256, size=(nblocks, 108), dtype=np.uint8)
    out[:, 108:110] = _fp16_scale_bytes(rng, nblocks, scale)
    return out.reshape(-1)


def pack_q4k_scales(scales: np.ndarray, mins: np.ndarray) -> np.ndarray:
    """[nb,8] 6-bit scales and mins -> [nb,12] packed bytes."""
    s = scales.astype(np.uint8)
    m = mins.astype(np.uint8)
    out = np.empty((s.shape[0], 12), dtype=np.uint8)
    out[:, 0:4] = (s[:, 0:4] & 63) | ((s[:, 4:8] >> 4) << 6)
    out[:, 4:8] = (m[:, 0:4] & 63) | ((m[:, 4:8] >> 4) << 6)
    out[:, 8:12] = (s[:, 4:8] & 15) | ((m[:, 4:8] & 15) << 4)
    return out


def q4_k_blocks(rng, nblocks: int, scale: float = 0.002) -> np.ndarray:
    out = np.empty((nblocks, 144), dtype=np.uint8)
    out[:, 0:2] = _fp16_scale_bytes(rng, nblocks, scale)
    out[:, 2:4] = _fp16_scale_bytes(rng, nblocks, scale)
    sc = rng.integers(0, 64, size=(nblocks, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(nblocks, 8), dtype=np.uint8)
    out[:, 4:16] = pack_q4k_scales(sc, mn)
    out[:, 16:144] = rng.integers(0, 256, size=(nblocks, 128), dtype=np.uint8)
    return out.reshape(-1)


def q5_k_blocks(rng, nblocks: int, scale: float = 0.002) -> np.ndarray:
    """Q5_K: as Q4_K plus 32 bytes of high bits (uniform), so the 5-bit codes are uniform 0..31."""
    out = np.empty((nblocks, 176), dtype=np.uint8)
    out[:, 0:2] = _fp16_scale_bytes(rng, nblocks, scale)
    out[:, 2:4] = _fp16_scale_bytes(rng, nblocks, scale)
    sc = rng.integers(0, 64, size=(nblocks, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(nblocks, 8), dtype=np.uint8)
    out[:, 4:16] = pack_q4k_scales(sc, mn)
    out[:, 16:176] = rng.integers(0, 256, size=(nblocks, 160), dtype=np.uint8)
    return out.reshape(-1)


def q6_k_blocks(rng, nblocks: int, scale: float = 0.0005) -> np.ndarray:
    out = np.empty((nblocks, 210), dtype=np.uint8)
    out[:, 0:192] = rng.integers(0, 256, size=(nblocks, 192), dtype=np.uint8)
    out[:, 192:208] = rng.integers(-64, 64, size=(nblocks, 16), dtype=np.int8).view(np.uint8)
    out[:, 208:210] = _fp16_scale_bytes(rng, nblocks, scale)
    return out.reshape(-1)


_GEN = {
    QuantFormat.Q4_0: q4_0_blocks,
    QuantFormat.Q8_0: q8_0_blocks,
    QuantFormat.Q4_K: q4_k_blocks,
    QuantFormat.Q5_K: q5_k_blocks,
    QuantFormat.Q5_0: q5_0_blocks,
    QuantFormat.Q2_K: q2_k_blocks,
    QuantFormat.Q3_K: q3_k_blocks,
    QuantFormat.Q6_K: q6_k_blocks,
}


def weight_bytes(fmt: QuantFormat, rng, n: int, k: int) -> np.ndarray:
    """Packed [N,K] weight (blocks along K) with the benchmark's value distribution."""
    fmt = QuantFormat.parse(fmt)
    assert k % fmt.block_size == 0
    return _GEN[fmt](rng, n * (k // fmt.block_size))


def device_weight(fmt, n: int, k: int, gen, device="cuda"):
    """The same distributions drawn ON THE DEVICE with torch's generator (for workloads too large to
    build on the host): every code byte uniform, Q6_K sub-scales uniform -64..63, Q4_K's twelve scale
    bytes uniform (which is exactly eight 6-bit scales and eight 6-bit mins uniform 0..63), block
    scales |N(0,1)| * c as fp16, Q4_K's d and dmin drawn independently.  Returns a ``QuantTensor``."""
    import torch

    from .tensor import QuantTensor

    f = QuantFormat.parse(fmt)
    nb = n * (k // f.block_size)
    w = torch.randint(0, 256, (nb, f.block_bytes), dtype=torch.uint8, device=device, generator=gen)
    c = {"Q4_0": 0.02, "Q5_0": 0.01, "Q8_0": 0.004, "Q2_K": 0.01, "Q3_K": 0.002, "Q4_K": 0.002, "Q5_K": 0.002, "Q6_K": 0.0005}[f.name]

    def scale():
        return (torch.randn(nb, device=device, generator=gen).abs() * c).to(torch.float16).view(torch.uint8).reshape(nb, 2)

    if f is QuantFormat.Q2_K:
        w[:, 80:82] = scale()
        w[:, 82:84] = scale()
    elif f is QuantFormat.Q3_K:
        w[:, 108:110] = scale()
    elif f is QuantFormat.Q6_K:
        w[:, 192:208] = torch.randint(-64, 64, (nb, 16), dtype=torch.int8, device=device, generator=gen).view(torch.uint8)
        w[:, 208:210] = scale()
    elif f is QuantFormat.Q8_0:
        w[:, 2:34] = torch.randint(-127, 128, (nb, 32), dtype=torch.int8, device=device, generator=gen).view(torch.uint8)
        w[:, 0:2] = scale()
    else:
        w[:, 0:2] = scale()
        if f in (QuantFormat.Q4_K, QuantFormat.Q5_K):
            w[:, 2:4] = scale()
    return QuantTensor(w.reshape(-1), f, (n, k))
