"""Q5_K on the GPU against the CPU oracle.

Two different element orders are at work in the reference and both are reproduced: ``dequantize`` follows
``dequant_q5k`` (src/quant/cpu/kernels/dequant_k_quants/q4k_q5k.rs:56-106, interleaved nibbles), the matmul
follows the Q8_K dot product x86-64 runs (src/quant/cpu/kernels/simd/fused_q5k_q8k_dot.rs:27-122, Q4_K's nibble
order).  Dequantised weights are bit-exact, matmul results agree to f32 summation order (integer dots are exact)."""
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

    return QuantTensor.from_bytes(w, F.Q5_K, (n, k), device="cuda")


@pytest.mark.parametrize("nblk", [1, 3, 17, 1000, 4099])
def test_dequant_bit_exact(ops, oracle, nblk):
    rng = synth.rng_for(70, nblk % 97)
    blocks = synth.q5_k_blocks(rng, nblk)
    from boostr_b200.tensor import QuantTensor

    qt = QuantTensor.from_bytes(blocks, F.Q5_K, (nblk * 256,), device="cuda")
    got = ops.dequantize(qt, torch.float32).cpu().numpy()
    want = oracle.dequantize_f32("Q5_K", blocks)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), describe_mismatch(got, want)
    bf = ops.dequantize(qt, torch.bfloat16).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(bf, oracle.dequantize_16("Q5_K", blocks, "bf16"))
    fh = ops.dequantize(qt, torch.float16).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(fh, oracle.dequantize_16("Q5_K", blocks, "f16"))
    assert np.array_equal(ops.dequantize(qt, torch.float64).cpu().numpy(), want.astype(np.float64))


@pytest.mark.parametrize("m,n,k", [(1, 1, 256), (1, 257, 2304), (1, 4096, 4096), (2, 33, 256), (5, 100, 4096), (8, 48, 4096),
                                   (16, 130, 4096), (4, 70, 14336), (12, 35, 14336), (33, 20, 512), (16, 14336, 4096)])
def test_matmul_small_m(ops, oracle, m, n, k):
    rng = synth.rng_for(71, seed_of(m, n, k))
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes("Q5_K", rng, n, k)
    guard = 4096
    flat = torch.full((2 * guard + m * n,), 4242.0, device="cuda")
    got = ops.quant_matmul(torch.from_numpy(act).cuda(), _qt(w, n, k), out=flat[guard:guard + m * n].view(m, n)).cpu().numpy()
    ops.check_device_status()
    assert torch.all(flat[:guard] == 4242.0) and torch.all(flat[guard + m * n:] == 4242.0)
    want = oracle.quant_matmul("Q5_K", act, w, n, threads=os.cpu_count() or 8, simd=True)
    e_max, e_rms = rel_err(got, want)
    assert e_max <= 2e-6, f"M={m} N={n} K={k}: max-norm err {e_max:.3e} rms {e_rms:.3e}\n" + describe_mismatch(got, want)


def test_swiglu_and_batch(ops, oracle):
    rng = synth.rng_for(72)
    m, n, k = 3, 96, 1024
    act = synth.activations(rng, m, k)
    wg, wu = synth.weight_bytes("Q5_K", rng, n, k), synth.weight_bytes("Q5_K", rng, n, k)
    got = ops.quant_swiglu(torch.from_numpy(act).cuda(), _qt(wg, n, k), _qt(wu, n, k)).cpu().numpy()
    want = oracle.quant_swiglu("Q5_K", act, wg, wu, n, threads=4)
    assert rel_err(got, want)[0] <= 1e-5
    from boostr_b200.tensor import QuantTensor

    w4 = synth.weight_bytes("Q4_K", rng, 64, k)
    outs = ops.quant_matmul_batch(torch.from_numpy(act).cuda(), [_qt(wg, n, k), QuantTensor.from_bytes(w4, "Q4_K", (64, k), device="cuda")])
    assert rel_err(outs[0].cpu().numpy(), oracle.quant_matmul("Q5_K", act, wg, n))[0] <= 2e-6
    assert rel_err(outs[1].cpu().numpy(), oracle.quant_matmul("Q4_K", act, w4, 64))[0] <= 2e-6


@pytest.mark.parametrize("m,n,k", [(64, 130, 512), (100, 257, 1024), (512, 1024, 4096)])
def test_prefill_tensor_core_path(ops, oracle, m, n, k):
    rng = synth.rng_for(73, seed_of(m, n, k))
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes("Q5_K", rng, n, k)
    got = ops.quant_matmul(torch.from_numpy(act).cuda(), _qt(w, n, k)).cpu().numpy()
    ops.check_device_status()
    want = oracle.quant_matmul("Q5_K", act, w, n, threads=os.cpu_count() or 8, simd=True)
    e_max, e_rms = rel_err(got, want)
    print(f"Q5_K prefill M={m} N={n} K={k}: vs CPU path max-norm {e_max:.2e} rms {e_rms:.2e}")
    assert e_max <= 1e-2, describe_mismatch(got, want)


def test_gguf_type_13_loads(ops, oracle, tmp_path):
    gguf = pytest.importorskip("gguf")
    from boostr_b200 import gguf as G

    rng = synth.rng_for(74)
    n, k = 64, 512
    w = synth.weight_bytes("Q5_K", rng, n, k)
    path = str(tmp_path / "q5.gguf")
    wr = gguf.GGUFWriter(path, "llama")
    wr.add_tensor("blk.0.ffn_down.weight", w.reshape(n, -1), raw_dtype=gguf.GGMLQuantizationType.Q5_K)
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    lin = G.load_llama_linears(path)["model.layers.0.mlp.down_proj"]
    assert lin.weight.format is F.Q5_K
    act = synth.activations(rng, 2, k)
    got = lin(torch.from_numpy(act).cuda()).cpu().numpy()
    assert rel_err(got, oracle.quant_matmul("Q5_K", act, w, n))[0] <= 2e-6
