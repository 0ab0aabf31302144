"""GPU parity: the CUDA library (through its C ABI) against the CPU oracle on the same seeded bytes.

Bars: dequantised weights bit-exact; matmul max|y - y_ref| / max|y_ref| <= 1e-3 for the
fp32-accumulate kernels (the tighter per-family bounds asserted below are what the design
is expected to reach) and <= 1e-2 for the bf16 tensor-core prefill path.
"""
import os

import numpy as np
import pytest

from boostr_b200 import synth
from boostr_b200.format import QuantError, QuantFormat as F
from util import describe_mismatch, rel_err, seed_of

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

FMTS = ["Q4_0", "Q8_0", "Q4_K", "Q6_K"]
GOLD = os.path.join(os.path.dirname(__file__), "golden", "dequant_witness.npz")


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from boostr_b200 import ops as o

    return o


def _qt(fmt, wbytes, n, k):
    from boostr_b200.tensor import QuantTensor

    return QuantTensor.from_bytes(wbytes, fmt, (n, k), device="cuda")


# ------------------------------------------------------------------ dequantize


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("nblk", [1, 3, 8, 17, 1000])
def test_dequant_f32_bit_exact(ops, oracle, fmt, nblk):
    f = F.parse(fmt)
    rng = synth.rng_for(20, f.value * 100 + nblk % 97)
    blocks = synth._GEN[f](rng, nblk)
    from boostr_b200.tensor import QuantTensor

    qt = QuantTensor.from_bytes(blocks, f, (nblk * f.block_size,), device="cuda")
    got = ops.dequantize(qt, torch.float32).cpu().numpy()
    want = oracle.dequantize_f32(fmt, blocks)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), describe_mismatch(got, want)


@pytest.mark.parametrize("fmt", FMTS)
def test_dequant_16bit_and_f64(ops, oracle, fmt):
    f = F.parse(fmt)
    nblk = 64 * (256 // f.block_size) + (3 if f.block_size == 32 else 0)
    rng = synth.rng_for(21, f.value)
    blocks = synth._GEN[f](rng, nblk)
    from boostr_b200.tensor import QuantTensor

    qt = QuantTensor.from_bytes(blocks, f, (nblk * f.block_size,), device="cuda")
    bf = ops.dequantize(qt, torch.bfloat16).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(bf, oracle.dequantize_16(fmt, blocks, "bf16"))
    fh = ops.dequantize(qt, torch.float16).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(fh, oracle.dequantize_16(fmt, blocks, "f16"))
    f64 = ops.dequantize(qt, torch.float64).cpu().numpy()
    assert np.array_equal(f64, oracle.dequantize_f32(fmt, blocks).astype(np.float64))


@pytest.mark.parametrize("fmt", FMTS)
def test_dequant_golden_witness(ops, fmt):
    g = np.load(GOLD)
    f = F.parse(fmt)
    blocks = g[f"{fmt}_blocks"]
    from boostr_b200.tensor import QuantTensor

    qt = QuantTensor.from_bytes(blocks, f, (blocks.size // f.block_bytes * f.block_size,), device="cuda")
    got = ops.dequantize(qt, torch.float32).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), g[f"{fmt}_f32"].view(np.uint32))


def test_dequant_full_size_checksum(ops, oracle):
    # Q4_K weight of BASELINE config 3 (14336 x 4096): every 997th block against the oracle,
    # plus linearity of the whole output in the block scale (size-independent property).
    f = F.Q4_K
    n, k = 14336, 4096
    rng = synth.rng_for(3, 1)
    w = synth.weight_bytes(f, rng, n, k)
    qt = _qt(f, w, n, k)
    got = ops.dequantize(qt, torch.bfloat16)
    blocks = w.reshape(-1, 144)
    pick = np.arange(0, blocks.shape[0], 997)
    want = oracle.dequantize_16("Q4_K", np.ascontiguousarray(blocks[pick]).reshape(-1), "bf16").reshape(len(pick), 256)
    g = got.view(torch.int16).reshape(-1, 256)[torch.from_numpy(pick).cuda()].cpu().numpy().view(np.uint16)
    assert np.array_equal(g, want)


def test_dequant_rejects_bad_target(ops):
    qt = _qt("Q8_0", synth.q8_0_blocks(synth.rng_for(22), 2), 2, 32)
    with pytest.raises(QuantError):
        ops.dequantize(qt, torch.int32)


# ------------------------------------------------------------------ quant_matmul (GEMV / small M)

SHAPES = [
    # (M, N, K)
    (1, 1, 256), (1, 17, 512), (2, 33, 256), (3, 64, 1024), (1, 257, 2304), (5, 100, 4096), (8, 48, 4096),
    (9, 40, 512), (16, 130, 4096), (1, 96, 8192), (4, 70, 14336), (12, 35, 14336), (17, 50, 1024), (33, 20, 512),
]


def _bound(fmt, m):
    if fmt in ("Q4_K", "Q6_K"):
        return 2e-6  # integer dots are exact; only the order of <= 56 f32 block terms differs
    # activations as int8 pieces: three pieces (22 bits) up to 8 rows, two pieces (15 bits) above
    return 1e-5 if m <= 8 else 1e-4


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_quant_matmul_small_m(ops, oracle, fmt, m, n, k):
    rng = synth.rng_for(23, (seed_of(fmt, m, n, k)))
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes(fmt, rng, n, k)
    # the output is the middle of one flat buffer: the guard regions before and after it must stay untouched
    guard = 4096
    flat = torch.full((2 * guard + m * n,), 12345.0, device="cuda")
    got_t = ops.quant_matmul(torch.from_numpy(act).cuda(), _qt(fmt, w, n, k), out=flat[guard:guard + m * n].view(m, n))
    ops.check_device_status()
    canary = torch.cat([flat[:guard], flat[guard + m * n:]])
    got = got_t.cpu().numpy()
    want = oracle.quant_matmul(fmt, act, w, n, threads=8)
    e_max, e_rms = rel_err(got, want)
    assert got.shape == (m, n)
    assert np.isfinite(got).all()
    assert e_max <= _bound(fmt, m), f"{fmt} M={m} N={n} K={k}: max-norm err {e_max:.3e} rms {e_rms:.3e}\n" + describe_mismatch(got, want)
    assert torch.all(canary == 12345.0)


@pytest.mark.parametrize("fmt", ["Q4_K", "Q6_K"])
def test_kquant_bit_exact_when_k_fits_one_chunk(ops, oracle, fmt):
    # K <= 4096: block terms are added in K order exactly as the CPU loop does
    rng = synth.rng_for(24, F.parse(fmt).value)
    m, n, k = 3, 77, 4096
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes(fmt, rng, n, k)
    got = ops.quant_matmul(torch.from_numpy(act).cuda(), _qt(fmt, w, n, k)).cpu().numpy()
    want = oracle.quant_matmul(fmt, act, w, n, threads=4)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), describe_mismatch(got, want)


@pytest.mark.parametrize("fmt", ["Q4_0", "Q8_0"])
@pytest.mark.parametrize("m,n,k", [(1, 1, 32), (2, 5, 96), (1, 40, 288), (9, 33, 4128)])
def test_ragged_k_for_32_blocks(ops, oracle, fmt, m, n, k):
    rng = synth.rng_for(25, k % 89 + m)
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes(fmt, rng, n, k)
    got = ops.quant_matmul(torch.from_numpy(act).cuda(), _qt(fmt, w, n, k)).cpu().numpy()
    ops.check_device_status()
    want = oracle.quant_matmul(fmt, act, w, n)
    e_max, _ = rel_err(got, want)
    assert e_max <= _bound(fmt, m), f"err {e_max:.3e}\n" + describe_mismatch(got, want)


def test_known_answers(ops):
    # the reference's closed-form cases (src/quant/cpu/kernels/quant_matmul.rs:415-510)
    def f16b(x):
        return np.array([x], np.float16).view(np.uint8)

    blk = np.zeros(18, np.uint8)
    blk[0:2] = f16b(2.0)
    blk[2:] = 0x99
    out = ops.quant_matmul(torch.ones(1, 32, device="cuda"), _qt("Q4_0", blk, 1, 32))
    assert out.shape == (1, 1) and abs(out.item() - 64.0) < 1e-4
    b8 = np.zeros(34, np.uint8)
    b8[0:2] = f16b(0.5)
    b8[2:] = 4
    act = torch.ones(2, 32, device="cuda")
    act[1] = 0.5
    out = ops.quant_matmul(act, _qt("Q8_0", b8, 1, 32)).cpu().numpy()
    assert abs(out[0, 0] - 64.0) < 1e-4 and abs(out[1, 0] - 32.0) < 1e-4
    b1 = blk.copy()
    b1[0:2] = f16b(1.0)
    b3 = blk.copy()
    b3[0:2] = f16b(3.0)
    out = ops.quant_matmul(torch.ones(1, 32, device="cuda"), _qt("Q4_0", np.concatenate([b1, b3]), 2, 32)).cpu().numpy()
    assert abs(out[0, 0] - 32.0) < 1e-4 and abs(out[0, 1] - 96.0) < 1e-4


def test_zero_activation_and_leading_dims(ops, oracle):
    rng = synth.rng_for(26)
    n, k = 40, 512
    w = synth.weight_bytes("Q4_K", rng, n, k)
    qt = _qt("Q4_K", w, n, k)
    z = ops.quant_matmul(torch.zeros(2, k, device="cuda"), qt)
    assert torch.all(z == 0)
    act = synth.activations(rng, 6, k)
    got = ops.quant_matmul(torch.from_numpy(act).cuda().reshape(2, 3, k), qt)
    assert got.shape == (2, 3, n)
    want = oracle.quant_matmul("Q4_K", act, w, n)
    assert rel_err(got.reshape(6, n).cpu().numpy(), want)[0] < 2e-6


def test_bf16_activation_extension(ops, oracle):
    rng = synth.rng_for(27)
    m, n, k = 4, 64, 1024
    act = synth.activations(rng, m, k)
    a_bf = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(act)).reshape(m, k)
    for fmt in FMTS:
        w = synth.weight_bytes(fmt, rng, n, k)
        got = ops.quant_matmul(torch.from_numpy(a_bf).cuda().to(torch.bfloat16), _qt(fmt, w, n, k)).cpu().numpy()
        want = oracle.quant_matmul(fmt, a_bf, w, n)  # oracle upcasts bf16 -> f32 exactly
        assert rel_err(got, want)[0] <= _bound(fmt, m), fmt


def test_run_twice_is_bitwise_identical(ops):
    rng = synth.rng_for(28)
    m, n, k = 7, 300, 4096
    act = torch.from_numpy(synth.activations(rng, m, k)).cuda()
    for fmt in FMTS:
        qt = _qt(fmt, synth.weight_bytes(fmt, rng, n, k), n, k)
        a = ops.quant_matmul(act, qt)
        b = ops.quant_matmul(act, qt)
        assert torch.equal(a, b), fmt


def test_argument_errors(ops):
    rng = synth.rng_for(29)
    qt = _qt("Q8_0", synth.weight_bytes("Q8_0", rng, 4, 64), 4, 64)
    with pytest.raises(QuantError, match="dimension mismatch"):
        ops.quant_matmul(torch.ones(2, 32, device="cuda"), qt)
    with pytest.raises(QuantError, match="must be F32"):
        ops.quant_matmul(torch.ones(2, 64, device="cuda", dtype=torch.float16), qt)
    from boostr_b200.tensor import QuantTensor

    with pytest.raises(QuantError, match="not a multiple"):
        QuantTensor.from_bytes(np.zeros(34, np.uint8), "Q8_0", (1, 33))
    with pytest.raises(QuantError, match="expected 34 bytes"):
        QuantTensor.from_bytes(np.zeros(35, np.uint8), "Q8_0", (1, 32))


# ------------------------------------------------------------------ swiglu / batch


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("m,n,k", [(1, 48, 512), (3, 130, 4096), (10, 64, 1024), (2, 40, 14336)])
def test_quant_swiglu(ops, oracle, fmt, m, n, k):
    rng = synth.rng_for(30, seed_of(fmt, m, n, k))
    act = synth.activations(rng, m, k)
    wg = synth.weight_bytes(fmt, rng, n, k)
    wu = synth.weight_bytes(fmt, rng, n, k)
    got = ops.quant_swiglu(torch.from_numpy(act).cuda(), _qt(fmt, wg, n, k), _qt(fmt, wu, n, k)).cpu().numpy()
    ops.check_device_status()
    want = oracle.quant_swiglu(fmt, act, wg, wu, n, threads=4)
    e_max, _ = rel_err(got, want)
    assert e_max <= max(_bound(fmt, m) * 4, 1e-5), f"err {e_max:.3e}\n" + describe_mismatch(got, want)


def test_quant_matmul_batch_mixed_formats(ops, oracle):
    rng = synth.rng_for(31)
    m, k = 2, 1024
    act = synth.activations(rng, m, k)
    specs = [("Q4_K", 64), ("Q4_K", 32), ("Q6_K", 32)]
    ws = [synth.weight_bytes(f, rng, n, k) for f, n in specs]
    outs = ops.quant_matmul_batch(torch.from_numpy(act).cuda(), [_qt(f, w, n, k) for (f, n), w in zip(specs, ws)])
    for (f, n), w, o in zip(specs, ws, outs):
        want = oracle.quant_matmul(f, act, w, n)
        assert rel_err(o.cpu().numpy(), want)[0] < 2e-6


@pytest.mark.parametrize("m", [3, 16, 40])
def test_small_m_batch_shares_the_activation_image(ops, m):
    # q, k (Q4_K), a Q5_K weight (reads the Q4_K image), v (Q6_K: its own image), then Q8_0 twice: consecutive weights of one
    # image format take ONE preparation launch; every output must have the bits of the separate call
    gen = torch.Generator(device="cuda")
    gen.manual_seed(17)
    k = 2048
    specs = [("Q4_K", 384), ("Q4_K", 96), ("Q5_K", 160), ("Q6_K", 96), ("Q8_0", 200), ("Q8_0", 72)]
    ws = [synth.device_weight(f, n, k, gen) for f, n in specs]
    x = torch.randn(m, k, device="cuda", generator=gen)
    single = []
    n_single = 0
    for w in ws:
        before = ops.launch_count()
        single.append(ops.quant_matmul(x, w).clone())
        n_single += ops.launch_count() - before
    before = ops.launch_count()
    outs = ops.quant_matmul_batch(x, ws)
    n_batch = ops.launch_count() - before
    ops.check_device_status()
    for a, b in zip(outs, single):
        assert torch.equal(a, b)
    # the images of weights 2, 3 and 6 were there already; at 40 rows the Q4_K weights take the integer tensor-core kernels
    # (their own image per call), so only the second Q8_0 weight finds its image
    assert n_batch == n_single - (3 if m <= 32 else 1), (n_batch, n_single)


# ------------------------------------------------------------------ BASELINE shapes


@pytest.mark.parametrize("fmt,m,n,k", [
    ("Q4_0", 1, 4096, 4096),      # config 1
    ("Q8_0", 1, 11008, 4096),     # config 2
    ("Q8_0", 8, 11008, 4096),
    ("Q8_0", 32, 11008, 4096),
    ("Q6_K", 1, 128256, 4096),    # config 4
    ("Q6_K", 16, 128256, 4096),
    ("Q4_K", 1, 14336, 4096),     # config 5 layer shapes
    ("Q6_K", 1, 4096, 14336),
    ("Q4_K", 16, 4096, 4096),
    ("Q6_K", 16, 4096, 14336),
    ("Q4_K", 32, 14336, 4096),
])
def test_baseline_shapes(ops, oracle, fmt, m, n, k):
    rng = synth.rng_for(2, seed_of(fmt, m, n))
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes(fmt, rng, n, k)
    got = ops.quant_matmul(torch.from_numpy(act).cuda(), _qt(fmt, w, n, k)).cpu().numpy()
    ops.check_device_status()
    want = oracle.quant_matmul(fmt, act, w, n, threads=os.cpu_count() or 8)
    e_max, e_rms = rel_err(got, want)
    print(f"{fmt} M={m} N={n} K={k}: max-norm {e_max:.2e} rms {e_rms:.2e}")
    assert e_max <= _bound(fmt, m), describe_mismatch(got, want)


# ------------------------------------------------------------------ prefill (M >= 64): tcgen05 tensor-core path

PREFILL_SHAPES = [(64, 128, 256), (64, 130, 512), (100, 257, 1024), (128, 384, 4096), (300, 200, 2048), (512, 1024, 4096)]


def _prepared_act(oracle, fmt, act):
    """bf16 activations as the tensor-core path builds them: K-quants quantise each 256-run to Q8_K
    (CPU oracle), multiply codes by the scale, then round to bf16; Q4_0/Q8_0 round the f32 values."""
    act = np.ascontiguousarray(act, dtype=np.float32)
    if fmt in ("Q4_K", "Q6_K"):
        q = oracle.quantize_q8k(act.reshape(-1)).reshape(-1, 292)
        d8 = q[:, 0:4].copy().view(np.float32)
        codes = q[:, 4:260].view(np.int8).astype(np.float32)
        act = (codes * d8).astype(np.float32).reshape(act.shape)
    return torch.from_numpy(oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(act)).reshape(act.shape)).cuda()


def _bf16_reference(ops, act_prepared, qt):
    """What the tensor-core path computes by construction: prepared bf16 activations x
    bf16(dequantised weights), f32 accumulate."""
    w = ops.dequantize(qt, torch.bfloat16).float()
    return (act_prepared.float() @ w.t()).cpu().numpy()


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("m,n,k", PREFILL_SHAPES)
def test_prefill_tensor_core_path(ops, oracle, fmt, m, n, k):
    rng = synth.rng_for(32, seed_of(fmt, m, n, k))
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes(fmt, rng, n, k)
    qt = _qt(fmt, w, n, k)
    act_t = torch.from_numpy(act).cuda()
    guard = 4096
    flat = torch.full((2 * guard + m * n,), 777.0, device="cuda")
    got = ops.quant_matmul(act_t, qt, out=flat[guard:guard + m * n].view(m, n)).cpu().numpy()
    ops.check_device_status()
    assert torch.all(flat[:guard] == 777.0) and torch.all(flat[guard + m * n:] == 777.0)
    assert got.shape == (m, n) and np.isfinite(got).all()
    # (1) the kernel against its own definition (tight): same bf16 operands, f32 accumulation
    ref_tc = _bf16_reference(ops, _prepared_act(oracle, fmt, act), qt)
    e_tc, _ = rel_err(got, ref_tc)
    assert e_tc <= 2e-5, f"{fmt} M={m} N={n} K={k}: vs bf16 reference {e_tc:.3e}\n" + describe_mismatch(got, ref_tc)
    # (2) against boostr's CPU path: the stated bound of the bf16 tensor-core path
    want = oracle.quant_matmul(fmt, act, w, n, threads=os.cpu_count() or 8)
    e_max, e_rms = rel_err(got, want)
    print(f"prefill {fmt} M={m} N={n} K={k}: vs CPU path max-norm {e_max:.2e} rms {e_rms:.2e}")
    assert e_max <= 1e-2, describe_mismatch(got, want)


def test_prefill_bf16_activations_and_outputs(ops, oracle):
    rng = synth.rng_for(33)
    m, n, k = 96, 256, 1024
    act = torch.from_numpy(synth.activations(rng, m, k)).cuda().to(torch.bfloat16)
    qt = _qt("Q4_K", synth.weight_bytes("Q4_K", rng, n, k), n, k)
    ref = _bf16_reference(ops, _prepared_act(oracle, "Q4_K", act.float().cpu().numpy()), qt)
    got = ops.quant_matmul(act, qt).cpu().numpy()
    assert rel_err(got, ref)[0] <= 2e-5
    got16 = ops.quant_matmul(act, qt, out_dtype=torch.bfloat16).float().cpu().numpy()
    assert rel_err(got16, ref)[0] <= 1e-2


def test_prefill_baseline_c3(ops, oracle):
    # config 3: Q4_K, K=4096, N=14336, bf16 activations; M=512 fully against the CPU path,
    # M=2048 against the bf16 definition plus 64 sampled columns against the CPU path
    rng = synth.rng_for(3, 2)
    n, k = 14336, 4096
    w = synth.weight_bytes("Q4_K", rng, n, k)
    qt = _qt("Q4_K", w, n, k)
    for m in (512, 2048):
        act = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(synth.activations(rng, m, k))).reshape(m, k)
        act_t = torch.from_numpy(act).cuda().to(torch.bfloat16)
        got = ops.quant_matmul(act_t, qt).cpu().numpy()
        ops.check_device_status()
        assert rel_err(got, _bf16_reference(ops, _prepared_act(oracle, "Q4_K", act), qt))[0] <= 2e-5
        cols = np.arange(0, n, n // 64)[:64] if m == 2048 else np.arange(0, n, 7)
        wsub = np.ascontiguousarray(w.reshape(n, -1)[cols]).reshape(-1)
        want = oracle.quant_matmul("Q4_K", act, wsub, len(cols), threads=os.cpu_count() or 8)
        e_max, e_rms = rel_err(got[:, cols], want)
        print(f"C3 M={m}: vs CPU path max-norm {e_max:.2e} rms {e_rms:.2e}")
        assert e_max <= 1e-2


@pytest.mark.parametrize("fmt,n,k", [("Q4_K", 4096, 4096), ("Q6_K", 4096, 14336), ("Q4_K", 14336, 4096)])
def test_prefill_c5_m64_layer_shapes(ops, oracle, fmt, n, k):
    # config 5 at 64 tokens per step: every linear of the stack takes the tensor-core path
    rng = synth.rng_for(5, seed_of(fmt, n, k))
    m = 64
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes(fmt, rng, n, k)
    got = ops.quant_matmul(torch.from_numpy(act).cuda(), _qt(fmt, w, n, k)).cpu().numpy()
    ops.check_device_status()
    want = oracle.quant_matmul(fmt, act, w, n, threads=os.cpu_count() or 8)
    e_max, e_rms = rel_err(got, want)
    print(f"C5 M=64 {fmt} N={n} K={k}: vs CPU path max-norm {e_max:.2e} rms {e_rms:.2e}")
    assert e_max <= 1e-2


@pytest.mark.parametrize("fmt", ["Q4_K", "Q8_0"])
def test_prefill_swiglu(ops, oracle, fmt):
    rng = synth.rng_for(34, F.parse(fmt).value)
    m, n, k = 80, 192, 1024
    act = synth.activations(rng, m, k)
    wg = synth.weight_bytes(fmt, rng, n, k)
    wu = synth.weight_bytes(fmt, rng, n, k)
    got = ops.quant_swiglu(torch.from_numpy(act).cuda(), _qt(fmt, wg, n, k), _qt(fmt, wu, n, k)).cpu().numpy()
    want = oracle.quant_swiglu(fmt, act, wg, wu, n, threads=4)
    assert rel_err(got, want)[0] <= 2e-2  # product of two 1e-2-class results


@pytest.mark.parametrize("m", [64, 200])
def test_prefill_batch_shares_prepared_activations(ops, m):
    # several weights against one activation matrix at large M: the weights of a class of formats (K-quants / the
    # others) reuse the activations the first of them prepared; every output must equal the single call's bits
    rng = synth.rng_for(36, m)
    k = 1024
    act = torch.from_numpy(synth.activations(rng, m, k)).cuda()
    spec = [("Q4_K", 512), ("Q4_K", 136), ("Q6_K", 136), ("Q8_0", 96), ("Q4_0", 64), ("Q5_K", 40), ("Q8_0", 300)]
    ws = [_qt(f, synth.weight_bytes(f, rng, n, k), n, k) for f, n in spec]
    outs = ops.quant_matmul_batch(act, ws)
    ops.check_device_status()
    for (f, n), w, o in zip(spec, ws, outs):
        one = ops.quant_matmul(act, w)
        assert torch.equal(o, one), (f, n)


# ------------------------------------------------------------------ tensor-parallel shard shapes (one GPU)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("m", [1, 16])
def test_tp_shard_shapes_of_the_decode_stack(ops, oracle, world, m):
    """Every per-rank linear of the Llama-3-8B-shaped stack at 2/4/8-way tensor parallelism (rows cut
    to 96 to keep the CPU side quick): K-split shards give 2-byte-aligned rows and odd slice counts."""
    rng = synth.rng_for(35, world * 100 + m)
    rows = 96
    for fmt, k in [("Q4_K", 4096), ("Q6_K", 4096), ("Q4_K", 4096 // world), ("Q6_K", 14336 // world)]:
        act = synth.activations(rng, m, k)
        w = synth.weight_bytes(fmt, rng, rows, k)
        got = ops.quant_matmul(torch.from_numpy(act).cuda(), _qt(fmt, w, rows, k)).cpu().numpy()
        ops.check_device_status()
        want = oracle.quant_matmul(fmt, act, w, rows, threads=4)
        e_max, _ = rel_err(got, want)
        assert e_max <= 2e-6, f"{fmt} K={k} M={m}: {e_max:.3e}\n" + describe_mismatch(got, want)
    k = 4096
    act = synth.activations(rng, m, k)
    wg = synth.weight_bytes("Q4_K", rng, rows, k)
    wu = synth.weight_bytes("Q4_K", rng, rows, k)
    got = ops.quant_swiglu(torch.from_numpy(act).cuda(), _qt("Q4_K", wg, rows, k), _qt("Q4_K", wu, rows, k)).cpu().numpy()
    want = oracle.quant_swiglu("Q4_K", act, wg, wu, rows, threads=4)
    assert rel_err(got, want)[0] <= 1e-5


def test_quant_matmul_batch_decode_fused_launch(ops, oracle):
    # M = 1: consecutive Q4_K weights, and a Q6_K weight right after them, share one launch (q/k/v-style);
    # odd row counts exercise segment boundaries inside a fill
    rng = synth.rng_for(36)
    k = 4096
    act = synth.activations(rng, 1, k)
    specs = [("Q4_K", 333), ("Q4_K", 50), ("Q4_K", 1024), ("Q6_K", 64), ("Q4_K", 70)]
    ws = [synth.weight_bytes(f, rng, n, k) for f, n in specs]
    before = ops.launch_count()
    outs = ops.quant_matmul_batch(torch.from_numpy(act).cuda(), [_qt(f, w, n, k) for (f, n), w in zip(specs, ws)])
    ops.check_device_status()
    assert ops.launch_count() - before == 2  # [Q4_K x3 + Q6_K] + [Q4_K]
    for (f, n), w, o in zip(specs, ws, outs):
        want = oracle.quant_matmul(f, act, w, n)
        assert o.shape == (1, n)
        assert rel_err(o.cpu().numpy(), want)[0] < 2e-6, (f, n)


@pytest.mark.parametrize("specs", [
    [("Q4_K", 4096), ("Q4_K", 1024), ("Q6_K", 1024)],   # q, k, v of the decode stack
    [("Q4_K", 2048), ("Q4_K", 512), ("Q6_K", 512)],     # the same on 2 ranks
    [("Q4_K", 7), ("Q6_K", 3)],
    [("Q4_K", 5000), ("Q6_K", 1)],
    [("Q4_K", 16), ("Q4_K", 16), ("Q4_K", 16), ("Q6_K", 6000)],
])
@pytest.mark.parametrize("k", [4096, 1024])
def test_quant_matmul_batch_decode_mixed_formats_one_launch(ops, oracle, specs, k):
    rng = synth.rng_for(38, k + len(specs) + specs[-1][1])
    act = synth.activations(rng, 1, k)
    ws = [synth.weight_bytes(f, rng, n, k) for f, n in specs]
    before = ops.launch_count()
    outs = ops.quant_matmul_batch(torch.from_numpy(act).cuda(), [_qt(f, w, n, k) for (f, n), w in zip(specs, ws)])
    ops.check_device_status()
    assert ops.launch_count() - before == 1
    for (f, n), w, o in zip(specs, ws, outs):
        want = oracle.quant_matmul(f, act, w, n)
        assert o.shape == (1, n)
        assert rel_err(o.cpu().numpy(), want)[0] < 2e-6, (f, n)


@pytest.mark.parametrize("fmt", ["Q4_K", "Q6_K"])
@pytest.mark.parametrize("k", [256, 512, 768, 1024, 1280, 2048, 2304])
@pytest.mark.parametrize("n", [1, 63, 64, 65, 1000, 4096])
def test_decode_short_rows_share_a_warp(ops, oracle, fmt, k, n):
    # K-split shards of a tensor-parallel group have few blocks per row: several rows then share a warp
    rng = synth.rng_for(39, k * 7 + n)
    act = synth.activations(rng, 1, k)
    w = synth.weight_bytes(fmt, rng, n, k)
    got = ops.quant_matmul(torch.from_numpy(act).cuda(), _qt(fmt, w, n, k)).cpu().numpy()
    ops.check_device_status()
    want = oracle.quant_matmul(fmt, act, w, n)
    e_max, _ = rel_err(got, want)
    assert e_max <= 2e-6, f"{fmt} K={k} N={n}: {e_max:.3e}\n" + describe_mismatch(got, want)


@pytest.mark.parametrize("k", [256, 1792, 3584, 4096, 4352, 7168, 14336])
@pytest.mark.parametrize("n", [1, 37, 500])
def test_q6k_decode_rows_of_any_alignment(ops, oracle, k, n):
    # Q6_K rows are 210 bytes per block: K-split shards (1792, 3584, 7168) and odd block counts give rows
    # that start on 2-, 4- or 8-byte boundaries only
    rng = synth.rng_for(37, k + n)
    act = synth.activations(rng, 1, k)
    w = synth.weight_bytes("Q6_K", rng, n, k)
    got = ops.quant_matmul(torch.from_numpy(act).cuda(), _qt("Q6_K", w, n, k)).cpu().numpy()
    ops.check_device_status()
    want = oracle.quant_matmul("Q6_K", act, w, n)
    e_max, _ = rel_err(got, want)
    assert e_max <= 2e-6, f"K={k} N={n}: {e_max:.3e}\n" + describe_mismatch(got, want)
