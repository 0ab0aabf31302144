"""Pins the CPU oracle: the reference's own known-answer tests, re-expressed, plus the
gguf-py witness fixture and SIMD-vs-scalar agreement.  No GPU needed."""
import os

import numpy as np
import pytest

from boostr_b200 import synth
from boostr_b200.format import QuantFormat as F
from util import seed_of

GOLD = os.path.join(os.path.dirname(__file__), "golden", "dequant_witness.npz")


def f16b(x):
    return np.array([x], dtype=np.float16).view(np.uint8)


# ---- dequant KATs: src/quant/cpu/kernels/dequant_simple.rs:185-211, :276-289 ----
def test_q4_0_zeros_and_known(oracle):
    blk = np.zeros(18, np.uint8)
    blk[0:2] = f16b(1.0)
    blk[2:] = 0x88
    assert np.all(oracle.dequantize_f32("Q4_0", blk) == 0.0)
    blk[0:2] = f16b(2.0)
    blk[2:] = 0x99
    assert np.all(oracle.dequantize_f32("Q4_0", blk) == 2.0)


def test_q4_0_interleaved_order(oracle):
    # out[2i] = low nibble of byte i, out[2i+1] = high nibble (dequant_simple.rs:24-31)
    blk = np.zeros(18, np.uint8)
    blk[0:2] = f16b(1.0)
    blk[2:] = np.arange(16, dtype=np.uint8) | (np.uint8(15) - np.arange(16, dtype=np.uint8)) << 4
    out = oracle.dequantize_f32("Q4_0", blk)
    assert np.array_equal(out[0::2], np.arange(16) - 8.0)
    assert np.array_equal(out[1::2], (15 - np.arange(16)) - 8.0)


def test_q8_0_known(oracle):
    blk = np.zeros(34, np.uint8)
    blk[0:2] = f16b(0.5)
    blk[2:] = 4
    assert np.all(oracle.dequantize_f32("Q8_0", blk) == 2.0)
    blk[2:] = np.uint8(256 - 6)
    assert np.all(oracle.dequantize_f32("Q8_0", blk) == -3.0)


# ---- q4k_q5k.rs:129-138, :181-190; q6k_q8k.rs:89-98 ----
def test_kquant_zero_blocks(oracle):
    assert np.all(oracle.dequantize_f32("Q4_K", np.zeros(144, np.uint8)) == 0.0)
    assert np.all(oracle.dequantize_f32("Q6_K", np.zeros(210, np.uint8)) == 0.0)


def test_q4k_scale_unpack_roundtrip(oracle):
    rng = np.random.default_rng(3)
    sc = rng.integers(0, 64, (5, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, (5, 8), dtype=np.uint8)
    packed = synth.pack_q4k_scales(sc, mn)
    # d = 1, dmin = 1, all nibbles 1 -> value = sc - mn, pins both unpack paths (i<4 and i>=4)
    blocks = np.zeros((5, 144), np.uint8)
    blocks[:, 0:2] = f16b(1.0)
    blocks[:, 2:4] = f16b(1.0)
    blocks[:, 4:16] = packed
    blocks[:, 16:] = 0x11
    out = oracle.dequantize_f32("Q4_K", blocks.reshape(-1)).reshape(5, 8, 32)
    want = sc.astype(np.float32) - mn.astype(np.float32)
    assert np.array_equal(out, np.broadcast_to(want[:, :, None], out.shape))
    sc0 = np.zeros(12, np.uint8)
    sc0[0], sc0[1] = 10, 20  # test_unpack_q4k_q5k_scales_basic
    b = np.zeros(144, np.uint8)
    b[0:2] = f16b(1.0)
    b[4:16] = sc0
    b[16:] = 0x11
    o = oracle.dequantize_f32("Q4_K", b)
    assert o[0] == 10.0 and o[32] == 20.0


def test_q6k_layout_by_hand(oracle):
    # one block decoded by an independent numpy restatement of q6k_q8k.rs:10-56
    rng = np.random.default_rng(11)
    blk = rng.integers(0, 256, 210, dtype=np.uint8)
    blk[208:210] = f16b(0.25)
    ql, qh = blk[:128].astype(np.int32), blk[128:192].astype(np.int32)
    sc = blk[192:208].view(np.int8).astype(np.float32)
    want = np.zeros(256, np.float32)
    for n in range(2):
        for l in range(32):
            is_ = l // 16
            h = qh[32 * n + l]
            q = [
                (ql[64 * n + l] & 15) | ((h & 3) << 4),
                (ql[64 * n + l + 32] & 15) | (((h >> 2) & 3) << 4),
                (ql[64 * n + l] >> 4) | (((h >> 4) & 3) << 4),
                (ql[64 * n + l + 32] >> 4) | (((h >> 6) & 3) << 4),
            ]
            for g in range(4):
                want[128 * n + 32 * g + l] = np.float32(0.25) * sc[8 * n + is_ + 2 * g] * np.float32(q[g] - 32)
    assert np.array_equal(oracle.dequantize_f32("Q6_K", blk), want)


@pytest.mark.parametrize("fmt", ["Q4_0", "Q8_0", "Q4_K", "Q6_K"])
def test_dequant_matches_gguf_witness(oracle, fmt):
    g = np.load(GOLD)
    got = oracle.dequantize_f32(fmt, g[f"{fmt}_blocks"])
    assert np.array_equal(got.view(np.uint32), g[f"{fmt}_f32"].view(np.uint32))


@pytest.mark.parametrize("fmt", ["Q4_0", "Q8_0", "Q4_K", "Q6_K"])
def test_dequant_16bit_is_rne_of_f32(oracle, fmt):
    g = np.load(GOLD)
    blocks = g[f"{fmt}_blocks"]
    f32 = oracle.dequantize_f32(fmt, blocks)
    assert np.array_equal(oracle.dequantize_16(fmt, blocks, "bf16"), oracle.f32_to_bf16_bits(f32))
    assert np.array_equal(oracle.dequantize_16(fmt, blocks, "f16"), f32.astype(np.float16).view(np.uint16))


# ---- quantize_act_q8k.rs:145-171 ----
def test_q8k_roundtrip_and_zeros(oracle):
    x = (np.arange(256, dtype=np.float32) - 128.0) * np.float32(0.1)
    q = oracle.quantize_q8k(x)
    d = q[0:4].view(np.float32)[0]
    assert d > 0
    codes = q[4:260].view(np.int8).astype(np.int32)
    bsums = q[260:292].view(np.int16)
    assert np.array_equal(bsums, codes.reshape(16, 16).sum(1))
    z = oracle.quantize_q8k(np.zeros(256, np.float32))
    assert z[0:4].view(np.float32)[0] == 0.0 and np.all(z[4:260] == 0)


def test_q8k_rounds_half_to_even(oracle):
    # amax = 127 -> id = 1: codes are rint(x); the x86 reference path is half-to-even
    x = np.zeros(256, np.float32)
    x[0] = 127.0
    x[1:7] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5]
    codes = oracle.quantize_q8k(x)[4:260].view(np.int8)
    assert list(codes[:7]) == [127, 0, 2, 2, 0, -2, -2]


def test_q8k_matches_numpy_model(oracle):
    rng = np.random.default_rng(5)
    x = rng.standard_normal(1024).astype(np.float32) * 3
    q = oracle.quantize_q8k(x).reshape(4, 292)
    for b in range(4):
        xb = x[256 * b:256 * b + 256]
        amax = np.abs(xb).max()
        d = np.float32(amax) / np.float32(127.0)
        idv = np.float32(127.0) / np.float32(amax)
        codes = np.clip(np.rint(xb * idv), -128, 127).astype(np.int8)
        assert q[b, 0:4].view(np.float32)[0] == d
        assert np.array_equal(q[b, 4:260].view(np.int8), codes)


# ---- matmul KATs: kernels/quant_matmul.rs:415-510, cpu/quant_matmul/tests.rs:19-88 ----
def test_matmul_q4_0_identity_like(oracle):
    blk = np.zeros(18, np.uint8)
    blk[0:2] = f16b(2.0)
    blk[2:] = 0x99
    out = oracle.quant_matmul("Q4_0", np.ones((1, 32), np.float32), blk, 1)
    assert out.shape == (1, 1) and out[0, 0] == 64.0


def test_matmul_q8_0_2x1(oracle):
    act = np.ones((2, 32), np.float32)
    act[1] = 0.5
    blk = np.zeros(34, np.uint8)
    blk[0:2] = f16b(0.5)
    blk[2:] = 4
    out = oracle.quant_matmul("Q8_0", act, blk, 1)
    assert out[0, 0] == 64.0 and out[1, 0] == 32.0


def test_matmul_multiple_output_cols(oracle):
    b0 = np.zeros(18, np.uint8)
    b0[0:2] = f16b(1.0)
    b0[2:] = 0x99
    b1 = b0.copy()
    b1[0:2] = f16b(3.0)
    out = oracle.quant_matmul("Q4_0", np.ones((1, 32), np.float32), np.concatenate([b0, b1]), 2)
    assert list(out[0]) == [32.0, 96.0]


def test_matmul_matches_dequant_matmul_q8_0(oracle):
    act = (np.arange(64, dtype=np.float32) * np.float32(0.1)).reshape(2, 32)
    rows = []
    for r in range(3):
        b = np.zeros(34, np.uint8)
        b[0:2] = f16b(0.5)
        b[2:] = r + 1
        rows.append(b)
    w = np.concatenate(rows)
    out = oracle.quant_matmul("Q8_0", act, w, 3)
    ref = act @ oracle.dequantize_f32("Q8_0", w).reshape(3, 32).T
    assert np.abs(out - ref).max() < 1e-2


def _q4k_block_large(blk):  # fused_q4k_q8k_dot.rs:212-226
    b = np.zeros(144, np.uint8)
    b[0:2] = f16b(0.8 + blk * 0.05)
    b[2:4] = f16b(0.1 + blk * 0.01)
    b[4:8] = blk % 10 + 1
    b[8:12] = blk % 5 + 1
    i = np.arange(16, 144)
    b[16:] = ((blk * 17 + i * 31) % 256).astype(np.uint8)
    return b


def _q6k_block_large(blk):  # fused_q6k_q8k_dot.rs:266-281
    b = np.zeros(210, np.uint8)
    b[208:210] = f16b(0.8 + blk * 0.05)
    b[192:208] = ((np.arange(16) % 7) - 3).astype(np.int8).view(np.uint8)
    b[0:128] = ((blk * 17 + np.arange(128) * 31) % 256).astype(np.uint8)
    b[128:192] = ((blk * 13 + np.arange(64) * 37) % 256).astype(np.uint8)
    return b


@pytest.mark.parametrize("fmt,mk", [("Q4_K", _q4k_block_large), ("Q6_K", _q6k_block_large)])
def test_q8k_dot_vs_f32_dot_reference_tolerance(oracle, fmt, mk):
    # the reference's own bound between its Q8_K integer path and dequant+dot: 2 % + 1.0
    k = 4096
    act = np.sin(np.arange(k, dtype=np.float32) * np.float32(0.003)).astype(np.float32)
    w = np.concatenate([mk(b) for b in range(16)])
    got = oracle.dot_q8k(fmt, oracle.quantize_q8k(act), w, k)
    ref = float(np.dot(act.astype(np.float64), oracle.dequantize_f32(fmt, w).astype(np.float64)))
    assert abs(got - ref) < abs(ref) * 0.02 + 1.0
    assert got == oracle.dot_q8k(fmt, oracle.quantize_q8k(act), w, k, simd=True)


def test_q4k_q8k_small_case(oracle):  # fused_q4k_q8k_dot.rs:181-209
    k = 256
    act = (np.arange(k, dtype=np.float32) - 128.0) * np.float32(0.01)
    w = np.zeros(144, np.uint8)
    w[0:2] = f16b(1.0)
    w[2:4] = f16b(0.5)
    w[4:8] = 0x03
    w[8:12] = 0x02
    w[12:16] = 0x10
    w[16:] = 0x73
    got = oracle.dot_q8k("Q4_K", oracle.quantize_q8k(act), w, k)
    ref = float(np.dot(act.astype(np.float64), oracle.dequantize_f32("Q4_K", w).astype(np.float64)))
    assert abs(got - ref) < abs(ref) * 0.02 + 1.0


# ---- whole-driver checks ----
@pytest.mark.parametrize("fmt", ["Q4_0", "Q8_0", "Q4_K", "Q6_K"])
@pytest.mark.parametrize("m,n,k", [(1, 5, 256), (3, 33, 512), (2, 64, 1024)])
def test_driver_thread_and_simd_invariance(oracle, fmt, m, n, k):
    rng = synth.rng_for(14, seed_of(fmt, m, n, k))
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes(fmt, rng, n, k)
    a = oracle.quant_matmul(fmt, act, w, n, threads=1, simd=False)
    b = oracle.quant_matmul(fmt, act, w, n, threads=4, simd=True)
    c = oracle.quant_matmul(fmt, act, w, n, threads=3, simd=True, lib="liboracle_scalar.so")
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert np.array_equal(a.view(np.uint32), c.view(np.uint32))


@pytest.mark.parametrize("fmt", ["Q4_0", "Q8_0", "Q4_K", "Q6_K"])
def test_driver_close_to_exact_math(oracle, fmt):
    rng = synth.rng_for(13, F.parse(fmt).value)
    m, n, k = 4, 96, 2048
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes(fmt, rng, n, k)
    got = oracle.quant_matmul(fmt, act, w, n, threads=2)
    ref = oracle.matmul_exact_f64(fmt, act, w, n)
    err = np.abs(got - ref).max() / np.abs(ref).max()
    # f32-activation formats agree to rounding; K-quants carry the Q8_K activation error (~1e-2)
    assert err < (3e-2 if fmt in ("Q4_K", "Q6_K") else 1e-5), err


def test_swiglu(oracle):
    rng = synth.rng_for(12)
    m, n, k = 2, 48, 512
    act = synth.activations(rng, m, k)
    wg = synth.weight_bytes("Q4_K", rng, n, k)
    wu = synth.weight_bytes("Q4_K", rng, n, k)
    g = oracle.quant_matmul("Q4_K", act, wg, n).astype(np.float64)
    u = oracle.quant_matmul("Q4_K", act, wu, n).astype(np.float64)
    want = g / (1 + np.exp(-g)) * u
    got = oracle.quant_swiglu("Q4_K", act, wg, wu, n)
    assert np.abs(got - want).max() <= 1e-6 * np.abs(want).max() + 1e-9


# ------------------------------------------------------------------ Q5_K (next-format row)


def _q5k_block(d, dmin, sc_bytes, qh_fill, qs_fill):
    blk = np.zeros(176, np.uint8)
    blk[0:2] = np.array([d], np.float16).view(np.uint8)
    blk[2:4] = np.array([dmin], np.float16).view(np.uint8)
    blk[4:16] = sc_bytes
    blk[16:48] = qh_fill
    blk[48:176] = qs_fill
    return blk


def test_q5k_reference_known_answers(oracle):
    # src/quant/cpu/kernels/dequant_k_quants/q4k_q5k.rs: test_dequant_q5k_zero, test_dequant_q5k_known_values
    assert np.all(oracle.dequantize_f32("Q5_K", np.zeros(176, np.uint8)) == 0)
    sc = np.zeros(12, np.uint8)
    sc[0:4] = 1
    out = oracle.dequantize_f32("Q5_K", _q5k_block(1.0, 0.0, sc, 0, 0x55))
    assert np.all(out[:128] == 5.0) and np.all(out[128:] == 0.0)
    # high bits set for every element: 5-bit code 16 + 5 = 21
    out = oracle.dequantize_f32("Q5_K", _q5k_block(1.0, 0.0, sc, 0xFF, 0x55))
    assert np.all(out[:128] == 21.0)


def test_q5k_dequant_layout_by_hand(oracle):
    # element 32 j + l takes nibble (l % 2) of qs[16 j + l / 2] and bit (idx % 8) of qh[idx / 8] (q4k_q5k.rs:76-100)
    rng = np.random.default_rng(5)
    from boostr_b200 import synth

    blk = synth.q5_k_blocks(rng, 3)
    got = oracle.dequantize_f32("Q5_K", blk).reshape(3, 256)
    for b in range(3):
        raw = blk.reshape(3, 176)[b]
        d = np.float32(raw[0:2].view(np.float16)[0])
        dmin = np.float32(raw[2:4].view(np.float16)[0])
        s = raw[4:16]
        scales = [int(s[i] & 63) if i < 4 else int((s[i + 4] & 15) | ((s[i - 4] >> 6) << 4)) for i in range(8)]
        mins = [int(s[i + 4] & 63) if i < 4 else int((s[i + 4] >> 4) | ((s[i] >> 6) << 4)) for i in range(8)]
        qh, qs = raw[16:48], raw[48:176]
        for j in range(8):
            for l in range(32):
                idx = 32 * j + l
                byte = int(qs[16 * j + l // 2])
                low = (byte & 15) if l % 2 == 0 else (byte >> 4)
                q = low | (((int(qh[idx // 8]) >> (idx % 8)) & 1) << 4)
                want = np.float32(np.float32(d * np.float32(scales[j])) * np.float32(q)) - np.float32(dmin * np.float32(mins[j]))
                assert got[b, idx] == np.float32(want), (b, j, l)


def test_q5k_q8k_dot_orders(oracle):
    """The reference's AVX2 Q5_K x Q8_K dot (what x86-64 runs) reads the nibbles in the Q4_K order, its scalar
    fallback in the interleaved order of its dequant: on bytes where the two orders differ they give different
    results, and only the scalar form agrees with `activation . dequantize(weight)` to Q8_K rounding.  Both are
    restated; the matmul oracle follows the AVX2 form."""
    from boostr_b200 import synth

    rng = np.random.default_rng(6)
    k = 1024
    w = synth.q5_k_blocks(rng, k // 256)
    act = rng.standard_normal(k).astype(np.float32)
    q8 = oracle.quantize_q8k(act)
    simd = oracle.dot_q8k("Q5_K", q8, w, k, simd=True)
    scal = oracle.dot_q8k("Q5_K", q8, w, k, simd=False)
    ref = float(act.astype(np.float64) @ oracle.dequantize_f32("Q5_K", w).astype(np.float64))
    assert abs(scal - ref) < 0.02 * abs(ref) + 1.0         # the reference's own tolerance (fused_q5k_q8k_dot.rs:288-292)
    assert abs(simd - scal) > 1e-3                          # the two forms really are different functions
    sc = np.zeros(12, np.uint8)
    sc[0:4], sc[4:8], sc[8:12] = 0x03, 0x02, 0x10
    a = ((np.arange(256) - 128) * 0.01).astype(np.float32)
    q8 = oracle.quantize_q8k(a)
    # when both nibbles of every byte are equal the two orders coincide
    same = _q5k_block(1.0, 0.5, sc, 0xAA, 0x55)
    assert oracle.dot_q8k("Q5_K", q8, same, 256, simd=True) == oracle.dot_q8k("Q5_K", q8, same, 256, simd=False)
    # the reference's own test block (fused_q5k_q8k_dot.rs:221-247) and its tolerance, for the form x86-64 runs
    blk = _q5k_block(1.0, 0.5, sc, 0xAA, 0x73)
    want = float(a.astype(np.float64) @ oracle.dequantize_f32("Q5_K", blk).astype(np.float64))
    assert abs(oracle.dot_q8k("Q5_K", q8, blk, 256, simd=True) - want) < abs(want) * 0.05 + 2.0


def test_q5k_matmul_driver_follows_the_avx2_form(oracle):
    from boostr_b200 import synth

    rng = np.random.default_rng(7)
    m, n, k = 3, 20, 512
    w = synth.weight_bytes("Q5_K", rng, n, k)
    act = rng.standard_normal((m, k)).astype(np.float32)
    out = oracle.quant_matmul("Q5_K", act, w, n, threads=2, simd=True)
    for i in range(m):
        q8 = oracle.quantize_q8k(act[i])
        for j in range(n):
            assert out[i, j] == np.float32(oracle.dot_q8k("Q5_K", q8, w.reshape(n, -1)[j].copy(), k, simd=True))


# ------------------------------------------------------------------ Q5_0 (src/quant/cpu/kernels/dequant_simple.rs:66-95)


def _q5_0_block(d, qh_fill, qs_fill):
    blk = np.zeros(22, dtype=np.uint8)
    blk[0:2] = f16b(d)
    blk[2:6] = qh_fill
    blk[6:22] = qs_fill
    return blk


def test_q5_0_known_values(oracle):  # dequant_simple.rs:230-257
    out = oracle.dequantize_f32("Q5_0", _q5_0_block(1.0, 0, 0))
    assert np.allclose(out, -16.0)
    out = oracle.dequantize_f32("Q5_0", _q5_0_block(1.0, 0xFF, 0))  # every high bit set, nibbles 0: code 16 -> 0
    assert np.allclose(out, 0.0)


def test_q5_0_order_and_numpy_model(oracle):
    # element 2 i = low nibble of byte i, element 2 i + 1 = its high nibble, element e takes bit e of the high-bit word
    rng = np.random.default_rng(50)
    w = synth.weight_bytes("Q5_0", rng, 7, 96)
    got = oracle.dequantize_f32("Q5_0", w)
    blocks = w.reshape(-1, 22)
    d = blocks[:, 0:2].copy().view(np.float16).astype(np.float32)[:, 0]
    qh = blocks[:, 2:6].copy().view(np.uint32)[:, 0]
    qs = blocks[:, 6:22]
    nib = np.empty((blocks.shape[0], 32), dtype=np.int32)
    nib[:, 0::2] = qs & 15
    nib[:, 1::2] = qs >> 4
    hb = (qh[:, None] >> np.arange(32, dtype=np.uint32)[None, :]) & 1
    want = ((nib | (hb.astype(np.int32) << 4)) - 16).astype(np.float32) * d[:, None]
    assert np.array_equal(got.reshape(-1, 32).view(np.uint32), want.view(np.uint32))


def test_q5_0_matmul_is_dequant_times_f32(oracle):
    # Q5_0 takes the dequantised-row path of quant_matmul_f32 (src/quant/cpu/kernels/quant_matmul.rs:193-209)
    rng = np.random.default_rng(51)
    m, n, k = 3, 9, 128
    w = synth.weight_bytes("Q5_0", rng, n, k)
    act = synth.activations(rng, m, k)
    got = oracle.quant_matmul("Q5_0", act, w, n, threads=2)
    deq = oracle.dequantize_f32("Q5_0", w).reshape(n, k).astype(np.float64)
    want = act.astype(np.float64) @ deq.T
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()


# ------------------------------------------------------------------ Q2_K (dequant_k_quants/q2k_q3k.rs:13-58, simd/fused_q2k_q8k_dot.rs)


def _q2k_numpy(w):
    """Independent restatement: element e = 128 n + 32 g + 16 h + l <- bits 2g..2g+1 of qs[32 n + 16 h + l], scale byte e // 16."""
    blocks = w.reshape(-1, 84)
    sc, qs = blocks[:, 0:16].astype(np.int32), blocks[:, 16:80].astype(np.int32)
    d = blocks[:, 80:82].copy().view(np.float16).astype(np.float32)[:, 0]
    dmin = blocks[:, 82:84].copy().view(np.float16).astype(np.float32)[:, 0]
    e = np.arange(256)
    n, g, h, l = e // 128, (e % 128) // 32, (e % 32) // 16, e % 16
    q = (qs[:, 32 * n + 16 * h + l] >> (2 * g)) & 3
    s = sc[:, e // 16]
    dl = d[:, None] * (s & 15).astype(np.float32)
    ml = dmin[:, None] * (s >> 4).astype(np.float32)
    return (dl * q.astype(np.float32)).astype(np.float32) - ml, q, s


def test_q2k_dequant_matches_numpy_model(oracle):
    rng = np.random.default_rng(60)
    w = synth.weight_bytes("Q2_K", rng, 5, 512)
    got = oracle.dequantize_f32("Q2_K", w).reshape(-1, 256)
    want, _, _ = _q2k_numpy(w)
    assert np.array_equal(got.view(np.uint32), want.astype(np.float32).view(np.uint32))


def test_q2k_zero_and_simple_blocks(oracle):
    blk = np.zeros(84, np.uint8)
    assert np.all(oracle.dequantize_f32("Q2_K", blk) == 0.0)
    blk[80:82] = f16b(1.0)   # d
    blk[82:84] = f16b(0.5)   # dmin
    blk[0:16] = 0x21         # scale 1, min 2
    blk[16:80] = 0xFF        # every code 3
    assert np.all(oracle.dequantize_f32("Q2_K", blk) == 3.0 - 1.0)


@pytest.mark.parametrize("mk", [(1, 256), (3, 1024)])
def test_q2k_q8k_dot_vs_f32_reference_tolerance(oracle, mk):  # fused_q2k_q8k_dot.rs:224-286: 2 % + 1.0
    m, k = mk
    rng = np.random.default_rng(61)
    n = 7
    w = synth.weight_bytes("Q2_K", rng, n, k)
    act = synth.activations(rng, m, k)
    got = oracle.quant_matmul("Q2_K", act, w, n, threads=2)
    ref = act.astype(np.float64) @ oracle.dequantize_f32("Q2_K", w).reshape(n, k).astype(np.float64).T
    assert np.all(np.abs(got - ref) <= 0.02 * np.abs(ref) + 1.0)
    # and tightly against an integer restatement of the same formula on the quantised activations
    _, q, s = _q2k_numpy(w)
    q = q.reshape(n, k // 256, 256)
    s = s.reshape(n, k // 256, 256)
    blocks = w.reshape(n, k // 256, 84)
    d = blocks[:, :, 80:82].copy().view(np.float16).astype(np.float32)[:, :, 0]
    dmin = blocks[:, :, 82:84].copy().view(np.float16).astype(np.float32)[:, :, 0]
    a = act.reshape(m, k // 256, 256)
    amax = np.abs(a).max(axis=2)
    idv = np.where(amax != 0, np.float32(127.0) / amax, 0).astype(np.float32)
    codes = np.clip(np.rint((a * idv[:, :, None]).astype(np.float32)), -128, 127).astype(np.int64)
    d8 = (amax / np.float32(127.0)).astype(np.float32)
    want = np.zeros((m, n), np.float32)
    for i in range(m):
        for j in range(n):
            acc = np.float32(0)
            for b in range(k // 256):
                isum = int(((s[j, b] & 15) * q[j, b] * codes[i, b]).sum())
                summs = int(((s[j, b] >> 4) * codes[i, b]).sum())
                t = np.float32(np.float32(d[j, b] * d8[i, b]) * np.float32(isum)) - np.float32(np.float32(dmin[j, b] * d8[i, b]) * np.float32(summs))
                acc = np.float32(acc + np.float32(t))
            want[i, j] = acc
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


# ------------------------------------------------------------------ Q3_K (dequant_k_quants/q2k_q3k.rs:64-144, simd/fused_q3k_q8k_dot.rs)


def _q3k_numpy(w):
    blocks = w.reshape(-1, 110)
    hm, qs, sc = blocks[:, 0:32].astype(np.int32), blocks[:, 32:96].astype(np.int32), blocks[:, 96:108]
    d = blocks[:, 108:110].copy().view(np.float16).astype(np.float32)[:, 0]
    # the reference's u32 unpacking, word by word (q2k_q3k.rs:115-144)
    aux = sc.copy().view(np.uint32).astype(np.uint64)
    a0, a1, tmp = aux[:, 0], aux[:, 1], aux[:, 2]
    k1, k2 = 0x03030303, 0x0F0F0F0F
    words = np.stack([(a0 & k2) | ((tmp & k1) << 4), (a1 & k2) | (((tmp >> 2) & k1) << 4),
                      ((a0 >> 4) & k2) | (((tmp >> 4) & k1) << 4), ((a1 >> 4) & k2) | (((tmp >> 6) & k1) << 4)], axis=1).astype(np.uint32)
    scales = words.view(np.uint8).reshape(-1, 16).astype(np.int32) - 32
    e = np.arange(256)
    n, g, hl = e // 128, (e % 128) // 32, e % 32
    low2 = (qs[:, 32 * n + hl] >> (2 * g)) & 3
    hbit = (hm[:, hl] >> (4 * n + g)) & 1
    code = low2 - np.where(hbit != 0, 0, 4)
    return d, scales, code


def test_q3k_dequant_matches_numpy_model(oracle):
    rng = np.random.default_rng(62)
    w = synth.weight_bytes("Q3_K", rng, 5, 512)
    got = oracle.dequantize_f32("Q3_K", w).reshape(-1, 256)
    d, scales, code = _q3k_numpy(w)
    want = (d[:, None] * scales[:, np.arange(256) // 16].astype(np.float32)).astype(np.float32) * code.astype(np.float32)
    assert np.array_equal(got.view(np.uint32), want.astype(np.float32).view(np.uint32))


def test_q3k_simple_blocks(oracle):
    blk = np.zeros(110, np.uint8)
    assert np.all(oracle.dequantize_f32("Q3_K", blk) == 0.0)
    blk[108:110] = f16b(1.0)
    blk[0:32] = 0xFF          # every high bit set: nothing subtracted
    blk[32:96] = 0xFF         # low bits 3
    blk[96:104] = 0x11        # low four bits of every scale: 1
    blk[104:108] = 0xAA       # high two bits: 2 -> scale (1 | 32) - 32 = 1
    assert np.all(oracle.dequantize_f32("Q3_K", blk) == 3.0)


def test_q3k_q8k_dot_forms(oracle):
    rng = np.random.default_rng(63)
    m, n, k = 2, 6, 768
    w = synth.weight_bytes("Q3_K", rng, n, k)
    act = synth.activations(rng, m, k)
    got = oracle.quant_matmul("Q3_K", act, w, n, threads=2)                 # the AVX2 form
    ref = act.astype(np.float64) @ oracle.dequantize_f32("Q3_K", w).reshape(n, k).astype(np.float64).T
    assert np.all(np.abs(got - ref) <= 0.02 * np.abs(ref) + 1.0)            # fused_q3k_q8k_dot.rs:300-364
    d, scales, code = _q3k_numpy(w)
    d, scales, code = d.reshape(n, -1), scales.reshape(n, -1, 16), code.reshape(n, -1, 256)
    a = act.reshape(m, k // 256, 256)
    amax = np.abs(a).max(axis=2)
    idv = np.where(amax != 0, np.float32(127.0) / amax, 0).astype(np.float32)
    codes8 = np.clip(np.rint((a * idv[:, :, None]).astype(np.float32)), -128, 127).astype(np.int64)
    d8 = (amax / np.float32(127.0)).astype(np.float32)
    want = np.zeros((m, n), np.float32)
    for i in range(m):
        for j in range(n):
            acc = np.float32(0)
            for b in range(k // 256):
                isum = int((scales[j, b][np.arange(256) // 16] * code[j, b] * codes8[i, b]).sum())
                acc = np.float32(acc + np.float32(np.float32(d[j, b] * d8[i, b]) * np.float32(isum)))
            want[i, j] = acc
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    scalar = oracle.quant_matmul("Q3_K", act, w, n, threads=2, simd=False)  # eight float lanes: close, not equal in general
    assert np.abs(scalar - got).max() <= 1e-5 * np.abs(got).max()


# ---- independent numpy restatements of the two Q8_K integer dot products, bit for bit against the C oracle ----
def _f16(b2):
    return np.frombuffer(bytes(b2), dtype=np.float16)[0].astype(np.float32)


def _q8k_numpy(x):
    """quantize_act_q8k.rs:26-98 for one row: per 256-block d8 (f32), 256 int8 codes, 16 sums of 16."""
    out = []
    for b in range(len(x) // 256):
        xb = x[256 * b:256 * b + 256]
        amax = np.float32(np.abs(xb).max())
        if amax == 0:
            out.append((np.float32(0), np.zeros(256, np.int32)))
            continue
        idv = np.float32(127.0) / amax
        codes = np.clip(np.rint(xb * idv), -128, 127).astype(np.int32)
        out.append((amax / np.float32(127.0), codes))
    return out


def _dot_q4k_numpy(row, q8):
    """fused_q4k_q8k_dot.rs:111-172: sumf += (d*d8)*sumi - (dmin*d8)*sumi_mins, block after block, no FMA."""
    acc = np.float32(0)
    for b, (d8, a) in enumerate(q8):
        blk = row[144 * b:144 * b + 144]
        d, dmin = _f16(blk[0:2]), _f16(blk[2:4])
        s = blk[4:16].astype(np.int32)
        sc = [s[j] & 63 if j < 4 else (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4) for j in range(8)]
        mn = [s[j + 4] & 63 if j < 4 else (s[j + 4] >> 4) | ((s[j] >> 6) << 4) for j in range(8)]
        qs = blk[16:144].astype(np.int32)
        sumi = 0
        summ = 0
        for jj in range(4):
            lo, hi = qs[32 * jj:32 * jj + 32] & 0xF, qs[32 * jj:32 * jj + 32] >> 4
            sumi += int(sc[2 * jj]) * int((lo * a[64 * jj:64 * jj + 32]).sum()) + int(sc[2 * jj + 1]) * int((hi * a[64 * jj + 32:64 * jj + 64]).sum())
            summ += int(mn[2 * jj]) * int(a[64 * jj:64 * jj + 32].sum()) + int(mn[2 * jj + 1]) * int(a[64 * jj + 32:64 * jj + 64].sum())
        term = (d * d8) * np.float32(sumi) - (dmin * d8) * np.float32(summ)
        acc = np.float32(acc + term)
    return acc


def _dot_q6k_numpy(row, q8):
    """fused_q6k_q8k_dot.rs:170-224: sumf += (d*d8)*sum_sb sc_sb * sum (q-32) a."""
    acc = np.float32(0)
    for b, (d8, a) in enumerate(q8):
        blk = row[210 * b:210 * b + 210]
        ql, qh = blk[0:128].astype(np.int32), blk[128:192].astype(np.int32)
        sc = blk[192:208].view(np.int8).astype(np.int32)
        d = _f16(blk[208:210])
        sumi = 0
        for n in range(2):
            for g in range(4):
                src = ql[64 * n + 32 * (g & 1):64 * n + 32 * (g & 1) + 32]
                nib = (src & 0xF) if g < 2 else (src >> 4)
                q = (nib | (((qh[32 * n:32 * n + 32] >> (2 * g)) & 3) << 4)) - 32
                e0 = 128 * n + 32 * g
                for half in range(2):
                    sumi += int(sc[8 * n + 2 * g + half]) * int((q[16 * half:16 * half + 16] * a[e0 + 16 * half:e0 + 16 * half + 16]).sum())
        acc = np.float32(acc + (d * d8) * np.float32(sumi))
    return acc


@pytest.mark.parametrize("fmt,dot", [("Q4_K", _dot_q4k_numpy), ("Q6_K", _dot_q6k_numpy)])
@pytest.mark.parametrize("simd", [True, False])
def test_kquant_dots_match_an_independent_numpy_restatement_bit_for_bit(oracle, fmt, dot, simd):
    m, n, k = 2, 6, 1024
    rng = synth.rng_for(41, 7 if fmt == "Q4_K" else 8)
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes(fmt, rng, n, k)  # the BASELINE distributions of the two formats
    got = oracle.quant_matmul(fmt, act, w, n, threads=1, simd=simd)
    rb = k // 256 * (144 if fmt == "Q4_K" else 210)
    want = np.empty((m, n), np.float32)
    for i in range(m):
        q8 = _q8k_numpy(act[i])
        for j in range(n):
            want[i, j] = dot(w[rb * j:rb * j + rb], q8)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (got, want)
