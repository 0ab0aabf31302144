"""The integer tensor-core small-M kernels (csrc/smallm_i8.cu: Q4_K, and Q8_0 above 16 rows) against the CPU oracle.

The Q4_K kernel takes every Q4_K product with 17..32 activation rows and, from 8 rows on, the matrices with enough 128-row tiles for
whole tiles per SM.  Bars: the integer sums are exact and the f32 block terms are added in K order, so a matrix that is
dealt in whole tiles has the oracle's BITS at any K the oracle adds in one chain (K <= 4096); a matrix whose tiles are
cut along K differs by the grouping of at most 56 f32 terms (<= 2e-6 of the largest output)."""
import os

import numpy as np
import pytest

from boostr_b200 import synth
from boostr_b200.format import QuantFormat as F
from util import describe_mismatch, rel_err, seed_of

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from boostr_b200 import ops as o

    return o


def _qt(w, n, k):
    from boostr_b200.tensor import QuantTensor

    return QuantTensor.from_bytes(w, F.Q4_K, (n, k), device="cuda")


def _threads():
    return os.cpu_count() or 8


# whole tiles per SM: 111 tiles and more on a 148-SM part, 8..16 rows; and every row count above 16
WHOLE = [(8, 14336, 4096), (16, 14336, 4096), (13, 14250, 2048), (32, 19000, 1024), (17, 128 * 148, 256), (16, 128256, 4096)]
# tiles cut along K (few tiles, or long K), ragged N, a single row of weights
CUT = [(17, 50, 1024), (24, 4096, 14336), (32, 1024, 4096), (20, 4096, 4096), (31, 1, 256), (18, 129, 512), (32, 300, 16384)]


@pytest.mark.parametrize("m,n,k", WHOLE)
def test_whole_tiles_have_the_oracles_bits(ops, oracle, m, n, k):
    rng = synth.rng_for(91, seed_of(m, n, k))
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes("Q4_K", rng, n, k)
    guard = 4096
    flat = torch.full((2 * guard + m * n,), 777.0, device="cuda")
    got = ops.quant_matmul(torch.from_numpy(act).cuda(), _qt(w, n, k), out=flat[guard:guard + m * n].view(m, n)).cpu().numpy()
    ops.check_device_status()
    assert (flat[:guard] == 777.0).all() and (flat[guard + m * n:] == 777.0).all(), "guard regions were written"
    want = oracle.quant_matmul("Q4_K", act, w, n, threads=_threads())
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), describe_mismatch(got, want)


@pytest.mark.parametrize("m,n,k", CUT)
def test_cut_tiles(ops, oracle, m, n, k):
    rng = synth.rng_for(92, seed_of(m, n, k))
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes("Q4_K", rng, n, k)
    guard = 4096
    flat = torch.full((2 * guard + m * n,), 777.0, device="cuda")
    x = torch.from_numpy(act).cuda()
    qt = _qt(w, n, k)
    got = ops.quant_matmul(x, qt, out=flat[guard:guard + m * n].view(m, n)).cpu().numpy()
    ops.check_device_status()
    assert (flat[:guard] == 777.0).all() and (flat[guard + m * n:] == 777.0).all(), "guard regions were written"
    want = oracle.quant_matmul("Q4_K", act, w, n, threads=_threads())
    e_max, e_rms = rel_err(got, want)
    assert np.isfinite(got).all()
    assert e_max <= 2e-6, f"M={m} N={n} K={k}: {e_max:.3e} (rms {e_rms:.3e})\n" + describe_mismatch(got, want)
    # the per-tile counters are back at zero: a second and a third call give the same bits
    for _ in range(2):
        again = ops.quant_matmul(x, qt).cpu().numpy()
        assert np.array_equal(again.view(np.uint32), got.view(np.uint32))
    ops.check_device_status()


def test_bf16_activations_and_16bit_outputs(ops, oracle):
    m, n, k = 24, 700, 2048
    rng = synth.rng_for(93, 1)
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes("Q4_K", rng, n, k)
    xb = torch.from_numpy(act).cuda().to(torch.bfloat16)
    act_bf = xb.float().cpu().numpy()
    want = oracle.quant_matmul("Q4_K", act_bf, w, n, threads=_threads())
    qt = _qt(w, n, k)
    got = ops.quant_matmul(xb, qt, out_dtype=torch.float32).cpu().numpy()
    assert rel_err(got, want)[0] <= 2e-6
    for dt, tol in ((torch.bfloat16, 2 ** -8), (torch.float16, 2 ** -10)):
        g16 = ops.quant_matmul(xb, qt, out_dtype=dt).float().cpu().numpy()
        assert rel_err(g16, want)[0] <= tol, dt
    ops.check_device_status()


@pytest.mark.parametrize("m,n,k", [(16, 14336, 4096), (32, 512, 1024), (19, 1000, 4096)])
def test_swiglu(ops, oracle, m, n, k):
    rng = synth.rng_for(94, seed_of(m, n, k))
    act = synth.activations(rng, m, k)
    wg = synth.weight_bytes("Q4_K", rng, n, k)
    wu = synth.weight_bytes("Q4_K", rng, n, k)
    got = ops.quant_swiglu(torch.from_numpy(act).cuda(), _qt(wg, n, k), _qt(wu, n, k)).cpu().numpy()
    ops.check_device_status()
    want = oracle.quant_swiglu("Q4_K", act, wg, wu, n, threads=_threads())
    e_max, _ = rel_err(got, want)
    assert e_max <= 1e-5, f"{e_max:.3e}\n" + describe_mismatch(got, want)


def test_zero_rows_and_a_zero_activation_row(ops, oracle):
    # an all-zero activation row quantises with d8 = 0 and must give exact zeros, beside ordinary rows
    m, n, k = 20, 260, 1024
    rng = synth.rng_for(95, 2)
    act = synth.activations(rng, m, k)
    act[7] = 0.0
    w = synth.weight_bytes("Q4_K", rng, n, k)
    got = ops.quant_matmul(torch.from_numpy(act).cuda(), _qt(w, n, k)).cpu().numpy()
    ops.check_device_status()
    want = oracle.quant_matmul("Q4_K", act, w, n, threads=4)
    assert (got[7] == 0.0).all()
    assert rel_err(got, want)[0] <= 2e-6


def test_graph_replay_is_bitwise_identical(ops):
    m, n, k = 32, 2048, 4096
    gen = torch.Generator(device="cuda")
    gen.manual_seed(9)
    w = synth.device_weight("Q4_K", n, k, gen)
    x = torch.randn(m, k, device="cuda", generator=gen)
    y = torch.empty(m, n, device="cuda")
    ref = ops.quant_matmul(x, w).clone()
    for _ in range(2):
        ops.quant_matmul(x, w, out=y)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        ops.quant_matmul(x, w, out=y)
    for _ in range(3):
        y.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(y, ref)
    ops.check_device_status()


# ------------------------------------------------------------------ Q8_0, 17..32 activation rows
# f32 activations on the CPU path; here two int8 pieces per value (relative error ~3e-5 of a 256-run's amax): the bar of
# the small-M kernel above 8 rows, 1e-4 of the largest output.

def _q8(w, n, k):
    from boostr_b200.tensor import QuantTensor

    return QuantTensor.from_bytes(w, F.Q8_0, (n, k), device="cuda")


@pytest.mark.parametrize("m,n,k", [(32, 11008, 4096), (17, 9600, 512), (24, 74 * 128 + 5, 1024), (31, 20000, 256)])
def test_q8_0_above_16_rows(ops, oracle, m, n, k):
    rng = synth.rng_for(96, seed_of(m, n, k))
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes("Q8_0", rng, n, k)
    guard = 4096
    flat = torch.full((2 * guard + m * n,), 555.0, device="cuda")
    x = torch.from_numpy(act).cuda()
    qt = _q8(w, n, k)
    got = ops.quant_matmul(x, qt, out=flat[guard:guard + m * n].view(m, n)).cpu().numpy()
    ops.check_device_status()
    assert (flat[:guard] == 555.0).all() and (flat[guard + m * n:] == 555.0).all(), "guard regions were written"
    want = oracle.quant_matmul("Q8_0", act, w, n, threads=_threads())
    e_max, e_rms = rel_err(got, want)
    assert np.isfinite(got).all()
    assert e_max <= 1e-4, f"M={m} N={n} K={k}: {e_max:.3e} (rms {e_rms:.3e})\n" + describe_mismatch(got, want)
    again = ops.quant_matmul(x, qt).cpu().numpy()
    assert np.array_equal(again.view(np.uint32), got.view(np.uint32))


def test_q8_0_swiglu_and_bf16(ops, oracle):
    m, n, k = 20, 9728, 1024
    rng = synth.rng_for(97, 3)
    act = synth.activations(rng, m, k)
    wg = synth.weight_bytes("Q8_0", rng, n, k)
    wu = synth.weight_bytes("Q8_0", rng, n, k)
    got = ops.quant_swiglu(torch.from_numpy(act).cuda(), _q8(wg, n, k), _q8(wu, n, k)).cpu().numpy()
    ops.check_device_status()
    want = oracle.quant_swiglu("Q8_0", act, wg, wu, n, threads=_threads())
    assert rel_err(got, want)[0] <= 4e-4
    xb = torch.from_numpy(act).cuda().to(torch.bfloat16)
    want_b = oracle.quant_matmul("Q8_0", xb.float().cpu().numpy(), wg, n, threads=_threads())
    got_b = ops.quant_matmul(xb, _q8(wg, n, k)).cpu().numpy()
    assert rel_err(got_b, want_b)[0] <= 1e-4


@pytest.mark.parametrize("fmt,m,n,k", [("Q4_K", 16, 14336, 4096), ("Q4_K", 32, 4096, 4096), ("Q4_K", 24, 4096, 14336), ("Q8_0", 32, 11008, 4096),
                                       ("Q4_K", 17, 1024, 4096)])
def test_many_replays_keep_their_bits_and_never_time_out(ops, fmt, m, n, k):
    # back-to-back launches (the next call's kernels start under programmatic dependent launch while this one drains):
    # every replay must reproduce the first result and no bounded wait may give up
    gen = torch.Generator(device="cuda")
    gen.manual_seed(11)
    ws = [synth.device_weight(fmt, n, k, gen) for _ in range(4)]
    x = torch.randn(m, k, device="cuda", generator=gen)
    y = torch.empty(m, n, device="cuda")
    ref = ops.quant_matmul(x, ws[-1]).clone()

    def run():
        for w in ws:
            ops.quant_matmul(x, w, out=y)

    run()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    for it in range(100):
        g.replay()
        if it % 20 == 19:
            torch.cuda.synchronize()
            assert torch.equal(y, ref)
    torch.cuda.synchronize()
    ops.check_device_status()


@pytest.mark.parametrize("fmt,m,n,k,tol", [("Q4_K", 40, 14336, 4096, 0.0), ("Q4_K", 63, 700, 1024, 2e-6), ("Q4_K", 33, 19000, 512, 0.0), ("Q8_0", 48, 11008, 1024, 1e-4),
                                           ("Q8_0", 33, 9600, 512, 1e-4)])
def test_33_to_63_rows_in_passes_of_32(ops, oracle, fmt, m, n, k, tol):
    # the bf16 tensor-core path starts at 64 rows; below it these rows go through the integer kernels in passes of up to 32
    # (a last pass of one row through the mma.sync kernel)
    from boostr_b200.tensor import QuantTensor

    rng = synth.rng_for(98, seed_of(fmt, m, n, k))
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes(fmt, rng, n, k)
    guard = 4096
    flat = torch.full((2 * guard + m * n,), 333.0, device="cuda")
    qt = QuantTensor.from_bytes(w, F.parse(fmt), (n, k), device="cuda")
    got = ops.quant_matmul(torch.from_numpy(act).cuda(), qt, out=flat[guard:guard + m * n].view(m, n)).cpu().numpy()
    ops.check_device_status()
    assert (flat[:guard] == 333.0).all() and (flat[guard + m * n:] == 333.0).all(), "guard regions were written"
    want = oracle.quant_matmul(fmt, act, w, n, threads=_threads())
    if tol == 0.0:
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), describe_mismatch(got, want)
    else:
        assert rel_err(got, want)[0] <= tol, describe_mismatch(got, want)
