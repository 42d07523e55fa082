"""The e4m3 block-scaled path (fused_experts with w1_scale / w2_scale / block_shape=[128, 128]).

The reference has no fp8 path, so there is nothing of its own to pin against: the checker is the CPU emulation of
the same quantisation scheme (oracle.fused_experts_fp8), itself tied to the bf16 oracle on dequantised weights.
Tolerances: rel-L2 <= 5e-3 against the emulation (same quantised operands, fp32 accumulation in another order);
rel-L2 <= 8e-2 against bf16 math on the dequantised weights (that distance is the activation quantisation:
e4m3 keeps 3 mantissa bits, and it is applied to x and to the intermediate)."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu

REL_L2_EMULATION = 5e-3
REL_L2_DEQUANT = 8e-2


def _dev():
    return torch.device("cuda", 0)


def _status_ok():
    from layered_prefill_b200 import ops
    assert ops.read_status(_dev()) == 0, "a device-side wait timed out"


@pytest.mark.parametrize("rows,cols", [(1, 128), (7, 256), (130, 2048), (64, 768)])
def test_activation_quantisation_is_bit_exact(rows, cols):
    from layered_prefill_b200 import fused_moe
    g = torch.Generator().manual_seed(rows + cols)
    x = (torch.randn(rows, cols, generator=g) * 3).to(torch.bfloat16)
    x[0, :128] = 0                      # an all-zero group: scale clamps at 1e-10 / 448
    if rows > 2:
        x[2, 5] = 1000.0                # one outlier sets its group's scale
    q, s = fused_moe.per_token_group_quant_fp8(x.to(_dev()))
    oq, os_ = O.per_token_group_quant_fp8(x)
    assert torch.equal(s.cpu(), os_)
    assert torch.equal(q.cpu().view(torch.uint8), oq.view(torch.uint8))


def _case(T, H, E, k, I, seed, skew=0.0, given_scales=False):
    from layered_prefill_b200 import fused_moe
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.02).to(torch.bfloat16)
    s13 = s2 = None
    if given_scales:  # the benchmark config's recipe: scales ~ U(0.5, 2) / 448, masters quantised with them
        s13 = (torch.rand(E, 2 * I // 128, H // 128, generator=g) * 1.5 + 0.5) / 448
        s2 = (torch.rand(E, H // 128, I // 128, generator=g) * 1.5 + 0.5) / 448
    q13, s13 = O.quant_weight_block_fp8(w13, s13)
    q2, s2 = O.quant_weight_block_fp8(w2, s2)
    logits = torch.randn(T, E, generator=g) + skew * torch.randn(E, generator=g)
    tw, ti, _ = O.fused_topk(x, logits, k, True)
    want = O.fused_experts_fp8(x, q13, s13, q2, s2, tw, ti)
    d = _dev()
    got = fused_moe.fused_experts(x.to(d), q13.to(d), q2.to(d), None, None, tw.to(d), ti.to(d), inplace=False,
                                  w1_scale=s13.to(d), w2_scale=s2.to(d), block_shape=[128, 128]).cpu()
    _status_ok()
    assert torch.isfinite(got.float()).all()
    assert O.rel_l2(got, want) <= REL_L2_EMULATION, (O.rel_l2(got, want), O.max_abs(got, want))
    deq = O.fused_experts(x, O.dequant_weight_block_fp8(q13, s13).to(torch.bfloat16),
                          O.dequant_weight_block_fp8(q2, s2).to(torch.bfloat16), tw, ti, "silu", "exact")
    assert O.rel_l2(got, deq) <= REL_L2_DEQUANT, O.rel_l2(got, deq)
    return got


@pytest.mark.parametrize("T,H,E,k,I", [
    (1, 128, 4, 1, 128),       # smallest legal shapes: one scale block everywhere
    (40, 256, 4, 2, 128),
    (130, 256, 8, 2, 256),     # more than one 128-row block per expert, two gate_up column tiles per half
    (64, 512, 16, 4, 384),     # three K blocks in the down pass
    (300, 384, 4, 2, 128),     # H = 3 scale blocks: odd number of stage products per tile
])
def test_fp8_experts_small_shapes(T, H, E, k, I):
    _case(T, H, E, k, I, seed=T + I)


def test_fp8_experts_imbalanced_routing_and_given_scales():
    _case(500, 256, 8, 2, 128, seed=9, skew=3.0, given_scales=True)


def test_fp8_experts_at_the_benchmark_width():
    """Qwen3-30B-A3B's H and I at decode size, a quarter of its experts (the CPU emulation quantises every weight)."""
    _case(64, 2048, 32, 8, 768, seed=11, given_scales=True)


def test_fp8_rejects_what_it_does_not_build():
    from layered_prefill_b200 import fused_moe
    d = _dev()
    x = torch.zeros(4, 192, dtype=torch.bfloat16, device=d)
    w13 = torch.zeros(2, 256, 192, dtype=torch.float8_e4m3fn, device=d)
    w2 = torch.zeros(2, 192, 128, dtype=torch.float8_e4m3fn, device=d)
    tw = torch.ones(4, 1, device=d)
    ti = torch.zeros(4, 1, dtype=torch.int32, device=d)
    with pytest.raises(ValueError):   # H not a multiple of 128
        fused_moe.fused_experts(x, w13, w2, None, None, tw, ti, w1_scale=torch.ones(2, 2, 2, device=d),
                                w2_scale=torch.ones(2, 2, 1, device=d), block_shape=[128, 128])
    with pytest.raises(ValueError):   # scales missing
        fused_moe.fused_experts(x, w13, w2, None, None, tw, ti)


def test_fp8_block_with_the_steps_in_front_replays_from_a_cuda_graph():
    """pre_moe (cluster kernel) + fp8 experts captured once and replayed on new inputs in the same buffers."""
    from layered_prefill_b200 import fused_moe
    g = torch.Generator().manual_seed(31)
    T, H, E, k, I = 48, 512, 128, 8, 128
    d = _dev()
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.02).to(torch.bfloat16)
    q13, s13 = O.quant_weight_block_fp8(w13)
    q2, s2 = O.quant_weight_block_fp8(w2)
    wg = (torch.randn(E, H, generator=g) * 0.05).to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    attn = [torch.randn(T, H, generator=g).to(torch.bfloat16) for _ in range(2)]
    res = [torch.randn(T, H, generator=g).to(torch.bfloat16) for _ in range(2)]
    a_buf, r_buf = attn[0].to(d), res[0].to(d)
    q13d, s13d, q2d, s2d, wgd, nwd = (t.to(d) for t in (q13, s13, q2, s2, wg, nw))

    def step():
        normed, _, tw, ti = fused_moe.pre_moe(a_buf, r_buf, nwd, 1e-6, wgd, k, True)
        return fused_moe.fused_experts(normed, q13d, q2d, None, None, tw, ti, inplace=False, w1_scale=s13d,
                                       w2_scale=s2d, block_shape=[128, 128])

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            r_buf.copy_(res[0])
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = step()
    for i in (1, 0):
        a_buf.copy_(attn[i])
        r_buf.copy_(res[i])
        graph.replay()
        torch.cuda.synchronize()
        normed, r_new = O.add_rms_norm(attn[i], res[i], nw, 1e-6)
        assert torch.equal(r_buf.cpu(), r_new)
        logits = O.router_gate(normed, wg)
        tw, ti, _ = O.fused_topk(normed, logits, k, True)
        want = O.fused_experts_fp8(normed, q13, s13, q2, s2, tw, ti)
        # the gate logits' summation order is free: on a near-tie the routing may differ from the CPU's, so the
        # comparison uses the tolerance of the dequantised path rather than the emulation's
        assert O.rel_l2(out.cpu(), want) <= REL_L2_DEQUANT
    _status_ok()


@pytest.mark.parametrize("T,H,E,k,I,tp,ranks", [
    (40, 256, 4, 2, 384, 2, (0, 1)),          # I/tp = 192: rank 1's slice starts in the middle of a scale block
    (130, 256, 8, 2, 768, 4, (0, 1, 2, 3)),   # slices [0,192) [192,384) [384,576) [576,768): shifts 0, 64, 0, 64
    (64, 512, 4, 4, 1536, 8, (0, 1, 6, 7)),   # the benchmark's 235B intermediate size at TP = 8
    (33, 256, 4, 2, 512, 2, (0, 1)),          # I/tp = 256: aligned slices take the same path with shift 0
])
def test_fp8_tensor_parallel_shards_use_the_unsharded_scale_blocks(T, H, E, k, I, tp, ranks):
    """One rank of a tensor-parallel fp8 layer on one GPU: weights sliced over I the way weight_loader slices them,
    scales of the unsharded tensors, the rank's partial sum against the CPU emulation of the same rank."""
    from layered_prefill_b200 import fused_moe
    g = torch.Generator().manual_seed(T + I + tp)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.03).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.03).to(torch.bfloat16)
    q13, s13 = O.quant_weight_block_fp8(w13)
    q2, s2 = O.quant_weight_block_fp8(w2)
    tw, ti, _ = O.fused_topk(x, torch.randn(T, E, generator=g), k, True)
    d = _dev()
    ip = I // tp
    parts = {}
    for r in ranks:
        q13r, q2r, lo = fused_moe.shard_fp8_expert_weights(q13, q2, r, tp)
        assert lo == r * ip
        want = O.fused_experts_fp8(x, q13r, s13, q2r, s2, tw, ti, i_offset=lo, i_total=I)
        got = fused_moe.fused_experts_fp8_shard(x.to(d), q13r.to(d), s13.to(d), q2r.to(d), s2.to(d), tw.to(d), ti.to(d),
                                                lo, I).cpu()
        _status_ok()
        assert torch.isfinite(got.float()).all()
        assert O.rel_l2(got, want) <= REL_L2_EMULATION, (r, O.rel_l2(got, want), O.max_abs(got, want))
        parts[r] = got
    if len(ranks) == tp:  # all ranks present: their sum is the layer's output, close to the unsharded emulation
        total = O.all_reduce([parts[r] for r in range(tp)])
        full = O.fused_experts_fp8(x, q13, s13, q2, s2, tw, ti)
        assert O.rel_l2(total, full) <= 3e-2   # a slice that splits a scale block quantises its halves separately


def test_fp8_experts_seeded_random_shapes():
    rng = torch.Generator().manual_seed(77)

    def pick(lo, hi, step=1):
        return int(torch.randint(lo // step, hi // step + 1, (1,), generator=rng).item()) * step

    for case in range(8):
        E = pick(2, 12)
        k = pick(1, min(E, 4))
        H = pick(128, 640, 128)
        I = pick(128, 512, 128)
        T = pick(1, 300)
        try:
            _case(T, H, E, k, I, seed=500 + case, skew=2.0 if case % 2 else 0.0, given_scales=case % 3 == 0)
        except AssertionError as err:
            raise AssertionError(f"case {case}: T={T} H={H} E={E} k={k} I={I}: {err}") from err
