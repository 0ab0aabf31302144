"""Q3_K on the GPU against the CPU oracle (dequant_q3k, src/quant/cpu/kernels/dequant_k_quants/q2k_q3k.rs:64-144; the
matmul follows fused_dot_q3k_q8k in the form x86-64 runs, src/quant/cpu/kernels/simd/fused_q3k_q8k_dot.rs:33-205, on
Q8_K-quantised activations).
Dequantised weights are bit-exact; matmul results are bit-identical for every M (integer sums, blocks added in K order)."""
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

    return QuantTensor.from_bytes(w, F.Q3_K, (n, k), device="cuda")


@pytest.mark.parametrize("nblk", [1, 3, 17, 1000, 4099])
def test_dequant_bit_exact(ops, oracle, nblk):
    rng = synth.rng_for(100, nblk % 97)
    blocks = synth.q3_k_blocks(rng, nblk)
    from boostr_b200.tensor import QuantTensor

    qt = QuantTensor.from_bytes(blocks, F.Q3_K, (nblk * 256,), device="cuda")
    got = ops.dequantize(qt, torch.float32).cpu().numpy()
    want = oracle.dequantize_f32("Q3_K", blocks)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), describe_mismatch(got, want)
    bf = ops.dequantize(qt, torch.bfloat16).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(bf, oracle.dequantize_16("Q3_K", blocks, "bf16"))
    assert np.array_equal(ops.dequantize(qt, torch.float64).cpu().numpy(), want.astype(np.float64))


@pytest.mark.parametrize("m,n,k", [(1, 1, 256), (1, 257, 2304), (1, 4096, 4096), (2, 33, 256), (5, 100, 4096), (9, 40, 512),
                                   (16, 130, 4096), (4, 70, 14336), (33, 20, 512), (70, 90, 1024)])
def test_matmul_bit_identical(ops, oracle, m, n, k):
    rng = synth.rng_for(101, seed_of(m, n, k))
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes("Q3_K", rng, n, k)
    guard = 4096
    flat = torch.full((2 * guard + m * n,), 4242.0, device="cuda")
    got = ops.quant_matmul(torch.from_numpy(act).cuda(), _qt(w, n, k), out=flat[guard:guard + m * n].view(m, n)).cpu().numpy()
    ops.check_device_status()
    assert (flat[:guard] == 4242.0).all() and (flat[guard + m * n:] == 4242.0).all(), "guard regions were written"
    want = oracle.quant_matmul("Q3_K", act, w, n, threads=os.cpu_count() or 8)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), describe_mismatch(got, want)


def test_swiglu_and_bf16_activations(ops, oracle):
    rng = synth.rng_for(102)
    m, n, k = 3, 96, 1024
    act = synth.activations(rng, m, k)
    wg, wu = synth.weight_bytes("Q3_K", rng, n, k), synth.weight_bytes("Q3_K", rng, n, k)
    got = ops.quant_swiglu(torch.from_numpy(act).cuda(), _qt(wg, n, k), _qt(wu, n, k)).cpu().numpy()
    want = oracle.quant_swiglu("Q3_K", act, wg, wu, n, threads=4)
    assert rel_err(got, want)[0] <= 1e-5
    ab = torch.from_numpy(act).cuda().to(torch.bfloat16)
    got = ops.quant_matmul(ab, _qt(wg, n, k)).cpu().numpy()
    want = oracle.quant_matmul("Q3_K", ab.float().cpu().numpy(), wg, n, threads=4)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
