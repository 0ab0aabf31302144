"""b200q_prefetch_next: the decode-loop hint that lets a single-row launch pull the head of the NEXT launch's weights into L2.
It has no counterpart in boostr (its decode step launches the linears back to back, src/model/llama/model/forward_graph.rs:22-73)
and must never change a result: every product is compared bit for bit with the same call made without a hint, for every
kernel that can consume one (Q4_K, Q4_K batch, Q4_K + Q6_K mixed, SwiGLU, Q6_K with one, two and four K-chunks) and every
kind of operation it can describe, including hints that no kernel can use."""
import pytest

from boostr_b200 import synth

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from boostr_b200 import ops as o

    return o


@pytest.fixture(scope="module")
def weights():
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0xFE7C)
    w = {
        "q": synth.device_weight("Q4_K", 4096, 4096, gen),
        "k": synth.device_weight("Q4_K", 1024, 4096, gen),
        "v": synth.device_weight("Q6_K", 1024, 4096, gen),
        "gate": synth.device_weight("Q4_K", 3000, 4096, gen),
        "up": synth.device_weight("Q4_K", 3000, 4096, gen),
        "down": synth.device_weight("Q6_K", 4096, 14336, gen),   # four K-chunks
        "down2": synth.device_weight("Q6_K", 600, 8192, gen),    # two K-chunks
        "short": synth.device_weight("Q4_K", 37, 1024, gen),     # fewer rows than SMs, short rows
        "o_shard8": synth.device_weight("Q4_K", 4096, 512, gen),     # row-parallel shards of an 8-rank group: two and
        "down_shard8": synth.device_weight("Q6_K", 4096, 1792, gen),  # seven blocks per row
        "q8": synth.device_weight("Q8_0", 512, 4096, gen),       # no streaming decode kernel: the hint is dropped
        "x4096": torch.randn(1, 4096, device="cuda", generator=gen),
        "x14336": torch.randn(1, 14336, device="cuda", generator=gen),
        "x8192": torch.randn(1, 8192, device="cuda", generator=gen),
        "x1024": torch.randn(1, 1024, device="cuda", generator=gen),
        "x512": torch.randn(1, 512, device="cuda", generator=gen),
        "x1792": torch.randn(1, 1792, device="cuda", generator=gen),
    }
    return w


# what the hinted-at operation may look like
NEXT = {
    "single_q4k": (["q"], False),
    "single_q6k": (["down"], False),
    "two_chunks": (["down2"], False),
    "batch_q4k": (["q", "k"], False),
    "mixed": (["q", "k", "v"], False),
    "swiglu": (["gate", "up"], True),
    "short": (["short"], False),
    "shard_q4k": (["o_shard8"], False),
    "shard_q6k": (["down_shard8"], False),
    "unusable": (["q8"], False),
}

# the call that consumes the hint
CALLS = {
    "matmul_q4k": lambda o, w: [o.quant_matmul(w["x4096"], w["q"])],
    "matmul_q6k_4chunks": lambda o, w: [o.quant_matmul(w["x14336"], w["down"])],
    "matmul_q6k_2chunks": lambda o, w: [o.quant_matmul(w["x8192"], w["down2"])],
    "matmul_q6k_1chunk": lambda o, w: [o.quant_matmul(w["x4096"], w["v"])],
    "matmul_short": lambda o, w: [o.quant_matmul(w["x1024"], w["short"])],
    "matmul_shard_q4k": lambda o, w: [o.quant_matmul(w["x512"], w["o_shard8"])],
    "matmul_shard_q6k": lambda o, w: [o.quant_matmul(w["x1792"], w["down_shard8"])],
    "batch_mixed": lambda o, w: o.quant_matmul_batch(w["x4096"], [w["q"], w["k"], w["v"]]),
    "batch_q4k": lambda o, w: o.quant_matmul_batch(w["x4096"], [w["q"], w["k"]]),
    "swiglu": lambda o, w: [o.quant_swiglu(w["x4096"], w["gate"], w["up"])],
    "matmul_q8_0": lambda o, w: [o.quant_matmul(w["x4096"], w["q8"])],   # cannot consume it: must drop it
}


@pytest.mark.parametrize("call", sorted(CALLS))
@pytest.mark.parametrize("nxt", sorted(NEXT))
def test_hint_never_changes_a_result(ops, weights, call, nxt):
    want = [t.clone() for t in CALLS[call](ops, weights)]
    names, swiglu = NEXT[nxt]
    ops.prefetch_next([weights[n] for n in names], swiglu=swiglu)
    got = CALLS[call](ops, weights)
    again = CALLS[call](ops, weights)  # the hint was for one call only
    torch.cuda.synchronize()
    ops.check_device_status()
    for a, b, c in zip(want, got, again):
        assert torch.equal(a, b), f"{call} after a {nxt} hint differs from the plain call"
        assert torch.equal(a, c)


def test_mlp_places_its_own_hint_and_keeps_the_callers(ops, weights):
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    down = synth.device_weight("Q6_K", 4096, 3072, gen)
    gate = synth.device_weight("Q4_K", 3072, 4096, gen)
    up = synth.device_weight("Q4_K", 3072, 4096, gen)
    want = ops.quant_mlp(weights["x4096"], gate, up, down).clone()
    ops.prefetch_next([weights["q"], weights["k"], weights["v"]])
    got = ops.quant_mlp(weights["x4096"], gate, up, down)
    torch.cuda.synchronize()
    ops.check_device_status()
    assert torch.equal(want, got)


def test_decode_stack_with_and_without_hints(ops):
    from boostr_b200.decode_graph import DecodeGraph
    from boostr_b200.decode_stack import DecodeStack

    st = DecodeStack(1, layers=3, vocab=32000)
    st.prefetch = False
    want = st.step().clone()
    st.prefetch = True
    got = st.step().clone()
    assert torch.equal(want, got)
    g = DecodeGraph(st.step, {"x": st.x}, {"logits": st.logits}).capture(warmup=2)
    for _ in range(3):
        out = g.replay()["logits"]
    torch.cuda.synchronize()
    ops.check_device_status()
    assert torch.equal(want, out)


def test_hint_argument_errors(ops, weights):
    import ctypes

    from boostr_b200 import _cabi

    L = _cabi.lib()
    fm = (ctypes.c_int * 1)(weights["q"].format.format_id)
    wp = (ctypes.c_void_p * 1)(weights["q"].storage.data_ptr())
    ns = (ctypes.c_size_t * 1)(4096)
    assert L.b200q_prefetch_next(7, 1, fm, wp, ns, 4096) == _cabi.ERR_INVALID_ARG          # unknown operation
    assert L.b200q_prefetch_next(_cabi.OP_QUANT_MATMUL, 0, fm, wp, ns, 4096) == _cabi.ERR_INVALID_ARG
    assert L.b200q_prefetch_next(_cabi.OP_QUANT_MATMUL, 1, None, wp, ns, 4096) == _cabi.ERR_INVALID_ARG
    bad = (ctypes.c_int * 1)(999)
    assert L.b200q_prefetch_next(_cabi.OP_QUANT_MATMUL, 1, bad, wp, ns, 4096) == _cabi.ERR_UNSUPPORTED_FORMAT
    odd = (ctypes.c_void_p * 1)(weights["q"].storage.data_ptr() + 2)
    assert L.b200q_prefetch_next(_cabi.OP_QUANT_MATMUL, 1, fm, odd, ns, 4096) == _cabi.ERR_INVALID_ARG
    # a SwiGLU hint needs gate and up of one shape; anything else is dropped without an error
    assert L.b200q_prefetch_next(_cabi.OP_QUANT_SWIGLU, 1, fm, wp, ns, 4096) == _cabi.OK
    want = ops.quant_matmul(weights["x4096"], weights["q"]).clone()
    assert torch.equal(want, ops.quant_matmul(weights["x4096"], weights["q"]))
