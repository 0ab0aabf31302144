"""b200q_quant_matmul_static_scratch: the entry point for hosts that cannot allocate scratch.

Such a caller — an FFI user whose runtime owns all device memory, or a path where cudaMalloc's
device-wide synchronisation is unacceptable — passes only inputs and outputs; what the kernels keep
between their phases (split-K partial sums, the prepared activation image of the small-M and
tensor-core paths) lives in an array inside the library.  The test drives the raw C ABI and requires the same
output as b200q_quant_matmul with caller-provided scratch, on two calls in a row (the array is
shared and keeps old contents, so the second call runs over the first call's leftovers).

Collected last (file name) so that a run stopping at the first failure has already run the rest;
it passes alone in a fresh process and after the other tests.
"""
import ctypes

import numpy as np
import pytest

from boostr_b200 import _cabi, synth
from boostr_b200.format import QuantFormat as F
from util import rel_err

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _run(lib, fmt, act_t, w_t, m, k, n, static):
    out = torch.full((m, n), float("nan"), device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    fid = F.parse(fmt).format_id
    if static:
        rc = lib.b200q_quant_matmul_static_scratch(fid, act_t.data_ptr(), _cabi.DT_F32, w_t.data_ptr(), out.data_ptr(),
                                                   _cabi.DT_F32, m, k, n, stream)
    else:
        need = lib.b200q_workspace_bytes(_cabi.OP_QUANT_MATMUL, fid, m, k, n)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        rc = lib.b200q_quant_matmul(fid, act_t.data_ptr(), _cabi.DT_F32, w_t.data_ptr(), out.data_ptr(), _cabi.DT_F32,
                                    m, k, n, ws.data_ptr(), ws.numel(), stream)
    assert rc == _cabi.OK, lib.b200q_last_error().decode()
    torch.cuda.synchronize()
    return out.cpu().numpy(), (lib.b200q_workspace_bytes(_cabi.OP_QUANT_MATMUL, fid, m, k, n))


@pytest.mark.parametrize("fmt,m,n,k", [("Q6_K", 12, 35, 14336), ("Q8_0", 3, 70, 8192), ("Q4_K", 1, 64, 4096),
                                       ("Q4_K", 128, 256, 4096)])   # the last one keeps a 1 MiB activation image in the array
def test_static_scratch_matches_caller_scratch_twice(fmt, m, n, k, oracle):
    assert torch.cuda.is_available()
    lib = _cabi.lib()
    rng = synth.rng_for(50, F.parse(fmt).value)
    results = []
    for call in range(2):  # second call: different data, same shared scratch
        act = synth.activations(rng, m, k)
        w = synth.weight_bytes(fmt, rng, n, k)
        act_t = torch.from_numpy(act).cuda()
        w_t = torch.from_numpy(w).cuda()
        ref, need = _run(lib, fmt, act_t, w_t, m, k, n, static=False)
        got, _ = _run(lib, fmt, act_t, w_t, m, k, n, static=True)
        assert np.isfinite(got).all()
        e_max, _ = rel_err(got, ref)
        assert e_max <= 1e-6, f"call {call}: {fmt} differs from the caller-scratch entry point by {e_max:.3e}"
        # and against the CPU path itself, so this test stands alone (tensor-core shapes: the bf16 bar)
        e_cpu, _ = rel_err(got, oracle.quant_matmul(fmt, act, w, n, threads=4))
        assert e_cpu <= (1e-2 if m >= 64 else 1e-5), f"call {call}: {fmt} vs the CPU path {e_cpu:.3e}"
        results.append(need)
    if (fmt, m) != ("Q4_K", 1):
        assert results[0] > 0, "this shape was chosen because it uses scratch"


def test_static_scratch_rejects_oversized_shape():
    lib = _cabi.lib()
    fid = F.Q8_0.format_id
    m, k, n = 16, 8192, 200000  # 2 * 16 * 200000 * 4 bytes of partial sums > 8 MiB
    assert lib.b200q_workspace_bytes(_cabi.OP_QUANT_MATMUL, fid, m, k, n) > _cabi.STATIC_SCRATCH_BYTES
    fake = ctypes.c_void_p(0x10000)  # never dereferenced: the size check comes first
    rc = lib.b200q_quant_matmul_static_scratch(fid, fake, _cabi.DT_F32, fake, fake, _cabi.DT_F32, m, k, n, None)
    assert rc == _cabi.ERR_WORKSPACE_TOO_SMALL
    msg = lib.b200q_last_error().decode()
    assert "needs" in msg and str(_cabi.STATIC_SCRATCH_BYTES) in msg
