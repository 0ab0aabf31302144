"""Q5_0 on the GPU against the CPU oracle (dequant_q5_0, src/quant/cpu/kernels/dequant_simple.rs:66-95; the matmul takes the
dequantised-row path of quant_matmul_f32 with f32 activations, src/quant/cpu/kernels/quant_matmul.rs:193-209).
Dequantised weights are bit-exact; the matmul keeps the bars of the other 32-element formats (int8 activation pieces:
1e-5 up to 8 rows, 1e-4 above; 1e-2 on the bf16 tensor-core path from 64 rows)."""
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

    return QuantTensor.from_bytes(w, F.Q5_0, (n, k), device="cuda")


@pytest.mark.parametrize("nblk", [1, 3, 8, 17, 1000, 32771])
def test_dequant_bit_exact(ops, oracle, nblk):
    rng = synth.rng_for(80, nblk % 97)
    blocks = synth.q5_0_blocks(rng, nblk)
    from boostr_b200.tensor import QuantTensor

    qt = QuantTensor.from_bytes(blocks, F.Q5_0, (nblk * 32,), device="cuda")
    got = ops.dequantize(qt, torch.float32).cpu().numpy()
    want = oracle.dequantize_f32("Q5_0", blocks)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), describe_mismatch(got, want)
    bf = ops.dequantize(qt, torch.bfloat16).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(bf, oracle.dequantize_16("Q5_0", blocks, "bf16"))
    assert np.array_equal(ops.dequantize(qt, torch.float64).cpu().numpy(), want.astype(np.float64))


@pytest.mark.parametrize("m,n,k", [(1, 1, 32), (1, 17, 512), (1, 257, 2304), (1, 4096, 4096), (2, 33, 256), (3, 64, 1056), (5, 100, 4096),
                                   (8, 48, 4096), (9, 40, 512), (16, 130, 4096), (4, 70, 14336), (17, 50, 1024), (33, 20, 512)])
def test_matmul_small_m(ops, oracle, m, n, k):
    rng = synth.rng_for(81, seed_of(m, n, k))
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes("Q5_0", rng, n, k)
    guard = 4096
    flat = torch.full((2 * guard + m * n,), 4242.0, device="cuda")
    got = ops.quant_matmul(torch.from_numpy(act).cuda(), _qt(w, n, k), out=flat[guard:guard + m * n].view(m, n)).cpu().numpy()
    ops.check_device_status()
    assert (flat[:guard] == 4242.0).all() and (flat[guard + m * n:] == 4242.0).all(), "guard regions were written"
    want = oracle.quant_matmul("Q5_0", act, w, n, threads=os.cpu_count() or 8)
    e_max, e_rms = rel_err(got, want)
    assert e_max <= (1e-5 if m <= 8 else 1e-4), f"M={m} N={n} K={k}: {e_max:.3e}\n" + describe_mismatch(got, want)


@pytest.mark.parametrize("m,n,k", [(64, 192, 1024), (80, 300, 4096), (200, 136, 2048 + 64), (512, 4096, 4096)])
def test_matmul_tensor_core_path(ops, oracle, m, n, k):
    rng = synth.rng_for(82, seed_of(m, n, k))
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes("Q5_0", rng, n, k)
    got = ops.quant_matmul(torch.from_numpy(act).cuda(), _qt(w, n, k)).cpu().numpy()
    ops.check_device_status()
    want = oracle.quant_matmul("Q5_0", act, w, n, threads=os.cpu_count() or 8)
    assert rel_err(got, want)[0] <= 1e-2
    # against bf16 weights x bf16 activations in f32: the kernel's own arithmetic
    wd = torch.from_numpy(oracle.dequantize_f32("Q5_0", w).reshape(n, k)).cuda().to(torch.bfloat16).float()
    ab = torch.from_numpy(act).cuda().to(torch.bfloat16).float()
    ref = (ab.double() @ wd.double().T).float().cpu().numpy()
    assert rel_err(got, ref)[0] <= 2e-5


def test_swiglu_and_batch(ops, oracle):
    rng = synth.rng_for(83)
    m, n, k = 4, 96, 1024
    act = synth.activations(rng, m, k)
    wg, wu = synth.weight_bytes("Q5_0", rng, n, k), synth.weight_bytes("Q5_0", rng, n, k)
    got = ops.quant_swiglu(torch.from_numpy(act).cuda(), _qt(wg, n, k), _qt(wu, n, k)).cpu().numpy()
    want = oracle.quant_swiglu("Q5_0", act, wg, wu, n, threads=4)
    assert rel_err(got, want)[0] <= 4e-5
    outs = ops.quant_matmul_batch(torch.from_numpy(act).cuda(), [_qt(wg, n, k), _qt(wu, n, k)])
    for o, w in zip(outs, (wg, wu)):
        assert rel_err(o.cpu().numpy(), oracle.quant_matmul("Q5_0", act, w, n, threads=4))[0] <= 1e-5
