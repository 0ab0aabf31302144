"""b200q_quant_mlp: the feed-forward block down(silu(gate x) * (up x)) of src/model/llama/model/blocks_mlp.rs:38-46 as one call.
It must give the bits of quant_swiglu followed by quant_matmul (it is those two, chained, with the hidden state in scratch)
and stay within the oracle's bound for the two products."""
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


def _qt(fmt, w, n, k):
    from boostr_b200.tensor import QuantTensor

    return QuantTensor.from_bytes(w, F.parse(fmt), (n, k), device="cuda")


@pytest.mark.parametrize("m", [1, 5, 20, 70])
@pytest.mark.parametrize("fgu,fdown", [("Q4_K", "Q6_K"), ("Q4_K", "Q4_K"), ("Q8_0", "Q8_0")])
def test_mlp_is_swiglu_then_down(ops, oracle, m, fgu, fdown):
    k, n_ff, n_out = 512, 1024, 300
    rng = synth.rng_for(99, seed_of(m, fgu, fdown))
    act = synth.activations(rng, m, k)
    wg = synth.weight_bytes(fgu, rng, n_ff, k)
    wu = synth.weight_bytes(fgu, rng, n_ff, k)
    wd = synth.weight_bytes(fdown, rng, n_out, n_ff)
    x = torch.from_numpy(act).cuda()
    qg, qu, qd = _qt(fgu, wg, n_ff, k), _qt(fgu, wu, n_ff, k), _qt(fdown, wd, n_out, n_ff)
    before = ops.launch_count()
    got = ops.quant_mlp(x, qg, qu, qd)
    launches = ops.launch_count() - before
    ops.check_device_status()
    two = ops.quant_matmul(ops.quant_swiglu(x, qg, qu), qd)
    assert torch.equal(got, two), "the chained call and the two separate calls differ"
    if m == 1 and fgu == "Q4_K":
        assert launches == 2, launches  # the fused SwiGLU decode kernel and the down projection's decode kernel
    h = oracle.quant_swiglu(fgu, act, wg, wu, n_ff, threads=8)
    want = oracle.quant_matmul(fdown, h, wd, n_out, threads=8)
    e_max, _ = rel_err(got.cpu().numpy(), want)
    # the hidden state differs from the oracle's by the silu of the GPU (and, from 64 rows on, by bf16 operands)
    assert e_max <= (3e-2 if m >= 64 else 1e-3), f"{e_max:.3e}\n" + describe_mismatch(got.cpu().numpy(), want)


def test_mlp_argument_errors(ops):
    from boostr_b200.format import QuantError

    gen = torch.Generator(device="cuda")
    gen.manual_seed(1)
    g = synth.device_weight("Q4_K", 512, 256, gen)
    u = synth.device_weight("Q4_K", 512, 256, gen)
    d_bad = synth.device_weight("Q4_K", 64, 256, gen)  # takes 256, the hidden state has 512
    x = torch.randn(2, 256, device="cuda", generator=gen)
    with pytest.raises(QuantError):
        ops.quant_mlp(x, g, u, d_bad)
