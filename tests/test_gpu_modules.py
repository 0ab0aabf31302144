"""GPU tests of the callers of the quantized ops: QuantLinear / MaybeQuantLinear (src/nn/linear.rs:60-179),
the column-/row-parallel linears and gather (src/distributed/tensor_parallel.rs:27-355) with a one-rank
group at M > 1, the GGUF loader feeding them, and the CUDA-graph decode loop."""
import os

import numpy as np
import pytest

from boostr_b200 import synth
from boostr_b200.format import QuantFormat as F
from util import rel_err

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from boostr_b200 import ops as o

    return o


def _qt(fmt, wbytes, n, k):
    from boostr_b200.tensor import QuantTensor

    return QuantTensor.from_bytes(wbytes, fmt, (n, k), device="cuda")


@pytest.mark.parametrize("fmt,m", [("Q4_K", 1), ("Q6_K", 5), ("Q8_0", 3), ("Q4_0", 70)])
def test_quant_linear_adds_bias_after_the_product(ops, oracle, fmt, m):
    from boostr_b200.linear import QuantLinear

    rng = synth.rng_for(40, F.parse(fmt).value + m)
    n, k = 96, 1024
    act = synth.activations(rng, m, k)
    w = synth.weight_bytes(fmt, rng, n, k)
    bias = rng.standard_normal(n, dtype=np.float32)
    lin = QuantLinear(_qt(fmt, w, n, k), torch.from_numpy(bias).cuda())
    assert lin.in_features == k and lin.out_features == n
    got = lin(torch.from_numpy(act).cuda()).cpu().numpy()
    want = oracle.quant_matmul(fmt, act, w, n) + bias[None, :]
    assert rel_err(got, want)[0] <= (1e-2 if m >= 64 else 1e-5)
    no_bias = QuantLinear(_qt(fmt, w, n, k))(torch.from_numpy(act).cuda()).cpu().numpy()
    assert np.array_equal(got, no_bias + bias[None, :])  # one f32 add per element, after the product


def test_forward_batch_with_and_without_biases(ops, oracle):
    from boostr_b200.linear import MaybeQuantLinear, QuantLinear

    rng = synth.rng_for(41)
    m, k = 1, 1024
    act = synth.activations(rng, m, k)
    act_t = torch.from_numpy(act).cuda()
    specs = [("Q4_K", 128), ("Q4_K", 64), ("Q6_K", 64)]
    ws = [synth.weight_bytes(f, rng, n, k) for f, n in specs]
    bias1 = rng.standard_normal(64, dtype=np.float32)
    plain = [QuantLinear(_qt(f, w, n, k)) for (f, n), w in zip(specs, ws)]
    before = ops.launch_count()
    outs = QuantLinear.forward_batch(plain, act_t)
    assert ops.launch_count() - before == 1          # bias-free and all quantized: one batched launch
    biased = [plain[0], QuantLinear(plain[1].weight, torch.from_numpy(bias1).cuda()), plain[2]]
    before = ops.launch_count()
    outs_b = QuantLinear.forward_batch(biased, act_t)
    assert ops.launch_count() - before == 3          # a bias anywhere: per-layer calls (linear.rs:160-178)
    for i, ((f, n), w) in enumerate(zip(specs, ws)):
        want = oracle.quant_matmul(f, act, w, n)
        assert rel_err(outs[i].cpu().numpy(), want)[0] < 2e-6
        assert rel_err(outs_b[i].cpu().numpy(), want + (bias1[None, :] if i == 1 else 0))[0] < 2e-6
    # MaybeQuantLinear: quantized arm delegates, dense arm is x @ W^T + b; a dense member disables the batch path
    dense_w = rng.standard_normal((32, k), dtype=np.float32)
    layers = [MaybeQuantLinear.from_weight(plain[0].weight), MaybeQuantLinear.standard(torch.from_numpy(dense_w).cuda())]
    assert layers[0].is_quantized and not layers[1].is_quantized
    ys = MaybeQuantLinear.forward_batch(layers, act_t)
    assert rel_err(ys[0].cpu().numpy(), oracle.quant_matmul("Q4_K", act, ws[0], 128))[0] < 2e-6
    assert rel_err(ys[1].cpu().numpy(), act @ dense_w.T)[0] < 1e-5
    ys2 = MaybeQuantLinear.forward_batch(layers[:1] + [MaybeQuantLinear.from_weight(plain[1].weight)], act_t)
    assert torch.equal(ys2[0], outs[0]) and torch.equal(ys2[1], outs[1])


@pytest.mark.parametrize("m", [4, 16])
def test_parallel_linears_with_a_one_rank_group(ops, oracle, m):
    """World size 1: the shards are the whole tensors, collectives are no-ops (as the reference's own tests
    run with NoOpCommunicator, tensor_parallel.rs:358-479); checks the M > 1 layout of gather_from_ranks and
    the P fake shards of a column split assembled by hand."""
    import torch.distributed as dist
    from boostr_b200.tensor_parallel import ColumnParallelQuantLinear, RowParallelQuantLinear, gather_from_ranks, scatter_to_rank

    created = False
    if not dist.is_initialized():
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29541", rank=0, world_size=1)
        created = True
    try:
        rng = synth.rng_for(42, m)
        n, k = 192, 2048
        act = synth.activations(rng, m, k)
        act_t = torch.from_numpy(act).cuda()
        for fmt in ("Q4_K", "Q6_K", "Q8_0"):
            w = synth.weight_bytes(fmt, rng, n, k)
            want = oracle.quant_matmul(fmt, act, w, n)
            bound = 2e-6 if fmt != "Q8_0" else 1e-3
            col = ColumnParallelQuantLinear.from_full(fmt, w, n, k, 0, 1)
            y = gather_from_ranks(col(act_t))
            assert y.shape == (m, n) and rel_err(y.cpu().numpy(), want)[0] <= bound
            row = RowParallelQuantLinear.from_full(fmt, w, n, k, 0, 1)
            assert rel_err(row(act_t).cpu().numpy(), want)[0] <= bound
            # four fake ranks on this GPU: column shards side by side give the row-major [M, N] result,
            # row shards' partial products add up to it
            parts = [ops.quant_matmul(act_t, scatter_to_rank(fmt, w, n, k, 0, r, 4)) for r in range(4)]
            assert rel_err(torch.cat(parts, dim=-1).cpu().numpy(), want)[0] <= bound
            kl = k // 4
            partial = sum(ops.quant_matmul(act_t[:, r * kl:(r + 1) * kl].contiguous(), scatter_to_rank(fmt, w, n, k, 1, r, 4)) for r in range(4))
            assert rel_err(partial.cpu().numpy(), want)[0] <= max(bound, 1e-5)
    finally:
        if created:
            dist.destroy_process_group()


def test_gguf_load_and_forward(ops, oracle, tmp_path):
    pytest.importorskip("gguf")
    from boostr_b200 import gguf as G
    from boostr_b200.linear import QuantLinear
    from boostr_b200.tensor_parallel import ColumnParallelQuantLinear, RowParallelQuantLinear
    from gguf_fixture import HID, write_gguf

    path = str(tmp_path / "m.gguf")
    packed = write_gguf(path, layers=1)
    rng = synth.rng_for(43)
    lin = G.load_llama_linears(path)
    assert set(lin) == {"lm_head"} | {f"model.layers.0.{s}" for s in (
        "self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")} | {
        f"model.layers.0.block_sparse_moe.experts.{i}.gate_proj" for i in range(5)}  # one tensor of every other format
    assert lin["model.layers.0.self_attn.q_proj"].bias is not None   # attn_q.bias rides along
    for m in (1, 6):
        for gname, (fmt, n, k, b) in packed.items():
            hf = G.gguf_to_hf_name(gname)[:-len(".weight")]
            layer = lin[hf]
            assert isinstance(layer, QuantLinear) and layer.weight.format is F.parse(fmt) and layer.weight.shape == (n, k)
            act = synth.activations(rng, m, k)
            got = layer(torch.from_numpy(act).cuda()).cpu().numpy()
            want = oracle.quant_matmul(fmt, act, b, n)
            if layer.bias is not None:
                want = want + layer.bias.cpu().numpy()[None, :]
            assert rel_err(got, want)[0] <= (2e-6 if fmt in ("Q4_K", "Q6_K") else 1e-5), (gname, m)
    # two ranks' shards loaded on this one GPU: column parts concatenate, row parts add up
    g = G.Gguf.open(path)
    shards = [G.GgufVarMap(g, "cuda", r, 2) for r in range(2)]
    act = synth.activations(rng, 3, HID)
    act_t = torch.from_numpy(act).cuda()
    fmt, n, k, b = packed["blk.0.attn_q.weight"]
    cols = [s.take_maybe_quant_linear("model.layers.0.self_attn.q_proj.weight", "model.layers.0.self_attn.q_proj.bias") for s in shards]
    assert all(isinstance(c, ColumnParallelQuantLinear) and c.weight.shape == (n // 2, k) for c in cols)
    want = oracle.quant_matmul(fmt, act, b, n) + lin["model.layers.0.self_attn.q_proj"].bias.cpu().numpy()[None, :]
    got = torch.cat([c(act_t) for c in cols], dim=-1).cpu().numpy()
    assert rel_err(got, want)[0] <= 2e-6
    fmt, n, k, b = packed["blk.0.attn_output.weight"]
    rows = [s.take_maybe_quant_linear("model.layers.0.self_attn.o_proj.weight") for s in shards]
    assert all(isinstance(r, RowParallelQuantLinear) and r.weight.shape == (n, k // 2) for r in rows)
    part = sum(ops.quant_matmul(act_t[:, r * (k // 2):(r + 1) * (k // 2)].contiguous(), rows[r].weight) for r in range(2))
    assert rel_err(part.cpu().numpy(), oracle.quant_matmul(fmt, act, b, n))[0] <= 1e-5


@pytest.mark.parametrize("m", [1, 4])
def test_decode_graph_replay_equals_eager(ops, m):
    """A captured step of the decode stack, replayed with new inputs, gives the bits of the eager step."""
    from boostr_b200.decode_graph import DecodeGraph, DeviceScalars
    from boostr_b200.decode_stack import DecodeStack

    stack = DecodeStack(m, layers=3, hidden=1024, kv=256, ffn=2048, vocab=4096, seed=7)
    scal = DeviceScalars(5)
    runner = DecodeGraph(stack.step, {"x": stack.x}, {"logits": stack.logits, "d": stack.d}, scalars=scal).capture()
    if m == 1:
        assert runner.launches_per_step == 3 * 4 + 1   # qkv batch, o, gate+up, down per layer; lm_head
    gen = torch.Generator(device="cuda")
    gen.manual_seed(11)
    for it in range(3):
        x = torch.randn(m, 1024, device="cuda", generator=gen)
        eager = {k: v.clone() for k, v in runner.run_eager(seq_len=5 + it, x=x).items()}
        stack.logits.zero_()
        stack.d.zero_()
        before = ops.launch_count()
        out = runner.replay(seq_len=5 + it, x=x)
        assert ops.launch_count() == before              # a replay issues no launches through the library
        ops.check_device_status()
        for k in eager:
            assert torch.equal(out[k], eager[k]), (it, k)
        assert int(scal.write_pos.item()) == 5 + it and int(scal.seq_len_k.item()) == 6 + it
    with pytest.raises(ValueError, match="shape"):
        runner.replay(x=torch.zeros(m + 1, 1024, device="cuda"))
    with pytest.raises(KeyError):
        runner.replay(y=torch.zeros(1, device="cuda"))


def _rmsnorm_np(x, g, eps):
    x = x.astype(np.float32)
    rs = np.float32(1.0) / np.sqrt((x * x).mean(axis=-1, keepdims=True, dtype=np.float32) + np.float32(eps))
    return (x * rs * g[None, :]).astype(np.float32)


@pytest.mark.parametrize("k,specs", [(4096, [("Q4_K", 512), ("Q4_K", 128), ("Q6_K", 128)]), (1024, [("Q4_K", 96)]),
                                     (8192, [("Q6_K", 64)]), (2048, [("Q6_K", 40), ("Q4_K", 33)])])
def test_rmsnorm_prologue_decode(ops, oracle, k, specs):
    """input_layernorm + batched projections as one operator, one activation row: the decode kernels normalise the row
    while they quantise it.  RMSNorm itself is numr's in the reference (source absent): the comparison is against
    x * (1 / sqrt(mean(x^2) + eps)) * w in f32 followed by the CPU path of the product; a last-bit difference in the
    normalised row can move a Q8_K code by one, hence the 1e-3 bar.  The fused form must also equal, bit for bit, the
    library's own unfused form (stand-alone normalisation launch, then the same product)."""
    from boostr_b200.tensor import QuantTensor

    rng = synth.rng_for(45, k + len(specs))
    act = synth.activations(rng, 1, k) * np.float32(3.0)
    g = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    ws = [synth.weight_bytes(f, rng, n, k) for f, n in specs]
    qts = [_qt(f, w, n, k) for (f, n), w in zip(specs, ws)]
    act_t, g_t = torch.from_numpy(act).cuda(), torch.from_numpy(g).cuda()
    before = ops.launch_count()
    outs = ops.rmsnorm_quant_matmul_batch(act_t, g_t, 1e-5, qts)
    fused_launches = ops.launch_count() - before
    ops.check_device_status()
    xn = _rmsnorm_np(act, g, 1e-5)
    for (f, n), w, o in zip(specs, ws, outs):
        want = oracle.quant_matmul(f, xn, w, n)
        assert rel_err(o.cpu().numpy(), want)[0] <= 1e-3, (f, n)
    # unfused form: a Q8_0 weight in the batch has no fused prologue, so the whole batch takes the stand-alone launch
    extra = QuantTensor.from_bytes(synth.weight_bytes("Q8_0", rng, 32, k), "Q8_0", (32, k), device="cuda")
    before = ops.launch_count()
    outs2 = ops.rmsnorm_quant_matmul_batch(act_t, g_t, 1e-5, qts + [extra])
    assert ops.launch_count() - before > fused_launches
    for a, b in zip(outs, outs2):
        assert torch.equal(a, b)
    want8 = oracle.quant_matmul("Q8_0", xn, extra_bytes := extra.storage.cpu().numpy(), 32)
    assert rel_err(outs2[-1].cpu().numpy(), want8)[0] <= 1e-4


@pytest.mark.parametrize("m", [4, 80])
def test_rmsnorm_prologue_more_rows(ops, oracle, m):
    rng = synth.rng_for(46, m)
    k = 1024
    act = synth.activations(rng, m, k)
    g = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    specs = [("Q4_K", 64), ("Q6_K", 48)]
    ws = [synth.weight_bytes(f, rng, n, k) for f, n in specs]
    outs = ops.rmsnorm_quant_matmul_batch(torch.from_numpy(act).cuda(), torch.from_numpy(g).cuda(), 1e-6,
                                          [_qt(f, w, n, k) for (f, n), w in zip(specs, ws)])
    ops.check_device_status()
    xn = _rmsnorm_np(act, g, 1e-6)
    for (f, n), w, o in zip(specs, ws, outs):
        assert rel_err(o.cpu().numpy(), oracle.quant_matmul(f, xn, w, n))[0] <= (1e-2 if m >= 64 else 1e-3)
