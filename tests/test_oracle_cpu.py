"""The CPU oracle against the reference-derived golden vectors and hand-checkable cases."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O


@pytest.mark.parametrize("name", ["route_a", "route_b", "route_c", "route_d"])
def test_routing_matches_reference_helper(golden, name):
    logits = torch.from_numpy(golden[f"{name}_logits"])
    k = golden[f"{name}_ids"].shape[1]
    w, ids, tei = O.topk_softmax(logits, k, renormalize=True)
    assert np.array_equal(ids.numpy(), golden[f"{name}_ids"])
    np.testing.assert_allclose(w.numpy(), golden[f"{name}_weights"], rtol=2e-6, atol=1e-7)
    T = logits.shape[0]
    assert np.array_equal(tei.numpy(), (np.arange(k)[None, :] * T + np.arange(T)[:, None]).astype(np.int32))


def test_routing_unnormalised_is_full_softmax(golden):
    logits = torch.from_numpy(golden["route_a_logits"])
    w, ids, _ = O.topk_softmax(logits, 8, renormalize=False)
    p = torch.softmax(logits, dim=-1)
    np.testing.assert_allclose(w.numpy(), torch.gather(p, 1, ids.long()).numpy(), rtol=3e-6, atol=1e-8)
    assert (w[:, :-1] >= w[:, 1:]).all()  # slots in descending probability


def test_routing_ties_go_to_lowest_index():
    logits = torch.zeros(3, 4)
    logits[1] = torch.tensor([1.0, 2.0, 2.0, 1.0])
    logits[2] = torch.tensor([5.0, 5.0, 5.0, 5.0])
    _, ids, _ = O.topk_softmax(logits, 2)
    assert ids.tolist() == [[0, 1], [1, 2], [0, 1]]


def test_routing_non_power_of_two():
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(11, 96, generator=g)
    w, ids, _ = O.topk_softmax(logits, 4, renormalize=False)
    p = torch.softmax(logits, -1)
    tv, ti = torch.topk(p, 4, dim=-1)
    assert torch.equal(ids.long(), ti)
    np.testing.assert_allclose(w.numpy(), tv.numpy(), rtol=3e-6)


def test_activation_and_sum_match_reference_helpers(golden):
    x = torch.from_numpy(golden["silu_in"])
    ours = O.silu_and_mul(x.to(torch.bfloat16)).float().numpy()
    np.testing.assert_allclose(ours, golden["silu_out"], rtol=2 ** -6, atol=1e-3)  # two bf16 roundings
    x = torch.from_numpy(golden["swiglu_in"])
    ours = O.swigluoai_and_mul(x.to(torch.bfloat16)).float().numpy()
    np.testing.assert_allclose(ours, golden["swiglu_out"], rtol=2 ** -7, atol=1e-3)
    c3 = torch.from_numpy(golden["sum_in"]).to(torch.bfloat16)
    assert np.array_equal(O.moe_sum(c3).float().numpy(), golden["sum_out"])  # bit-exact


def _align_by_hand(ids, bs, E):
    ids = ids.reshape(-1).tolist()
    numel = len(ids)
    out, eids = [], []
    for e in range(E):
        mine = [i for i, v in enumerate(ids) if v == e]
        if not mine:
            continue
        pad = (-len(mine)) % bs
        out += mine + [numel] * pad
        eids += [e] * ((len(mine) + pad) // bs)
    return out, eids


@pytest.mark.parametrize("T,k,E,bs", [(3, 2, 4, 4), (17, 2, 8, 16), (64, 8, 128, 16), (5, 1, 3, 1), (40, 4, 16, 128)])
def test_align_against_hand_rolled(T, k, E, bs):
    g = torch.Generator().manual_seed(T * 131 + E)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    s, e, post = O.moe_align_block_size(ids, bs, E)
    hs, he = _align_by_hand(ids, bs, E)
    assert int(post) == len(hs)
    assert s[:len(hs)].tolist() == hs
    assert (s[len(hs):] == T * k).all()
    assert e[:len(he)].tolist() == he
    assert (e[len(he):] == 0).all()
    assert s.numel() == T * k + E * (bs - 1)


def test_align_edge_cases():
    # an expert with exactly block_size tokens, one with none, ids out of range are skipped
    ids = torch.tensor([[0, 2], [0, 2], [0, 3], [0, 7]], dtype=torch.int32)
    s, e, post = O.moe_align_block_size(ids, 4, 4)
    assert int(post) == 12
    assert s[:12].tolist() == [0, 2, 4, 6, 1, 3, 8, 8, 5, 8, 8, 8]
    assert e[:3].tolist() == [0, 2, 3]
    s, e, post = O.moe_align_block_size(torch.zeros(0, 2, dtype=torch.int32), 4, 4)
    assert int(post) == 0 and (s == 0).all()


def test_canonicalize_is_order_free():
    ids = torch.tensor([[1, 0], [1, 0], [0, 1]], dtype=torch.int32)
    s, e, post = O.moe_align_block_size(ids, 4, 2)
    shuffled = s.clone()
    shuffled[0:3] = s[[2, 0, 1]]
    c = O.canonicalize_sorted_ids(shuffled, e, int(post), 4, 6)
    assert torch.equal(c, s)


def test_expert_loop_matches_dense_formula():
    g = torch.Generator().manual_seed(0)
    T, H, E, k, I = 9, 32, 4, 2, 16
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.2).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.2).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    tw, ti, _ = O.fused_topk(x, logits, k, True)
    got = O.fused_experts(x, w13, w2, tw, ti, mode="exact").float()
    want = torch.zeros(T, H)
    for t in range(T):
        for j in range(k):
            e = int(ti[t, j])
            c1 = x[t].float() @ w13[e].float().t()
            h = torch.nn.functional.silu(c1[:I]) * c1[I:]
            want[t] += tw[t, j] * (h @ w2[e].float().t())
    assert O.rel_l2(got, want) < 4e-3  # one bf16 rounding of the output
    ref = O.fused_experts(x, w13, w2, tw, ti, mode="ref_rounding").float()
    assert O.rel_l2(ref, want) < 2e-2


@pytest.mark.parametrize("tp", [2, 4, 8])
def test_tp_shards_sum_to_full_block(tp):
    """Sum over ranks of block(I-slice) == block(full I): the sharding of layers/fused_moe.py:398-432."""
    g = torch.Generator().manual_seed(1)
    T, H, E, k, I = 12, 64, 8, 2, 128
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.1).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.1).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    tw, ti, _ = O.fused_topk(x, logits, k, True)
    full = O.fused_experts(x, w13, w2, tw, ti, mode="exact").float()
    parts = [O.fused_experts(x, *O.shard_expert_weights(w13, w2, tp, r), tw, ti, mode="exact").float()
             for r in range(tp)]
    assert O.rel_l2(sum(parts), full) < 6e-3
    sh13, sh2 = O.shard_expert_weights(w13, w2, tp, 1)
    assert sh13.shape == (E, 2 * I // tp, H) and sh2.shape == (E, H, I // tp)
    assert torch.equal(sh13[:, :I // tp], w13[:, I // tp:2 * I // tp])
    assert torch.equal(sh13[:, I // tp:], w13[:, I + I // tp:I + 2 * I // tp])


def test_all_reduce_order_and_single_rounding():
    a = torch.tensor([1.0, 256.0]).to(torch.bfloat16)
    b = torch.tensor([2.0 ** -9, 1.0]).to(torch.bfloat16)
    c = torch.tensor([2.0 ** -9, 1.0]).to(torch.bfloat16)
    out = O.all_reduce([a, b, c])
    # fp32 accumulation keeps the two small addends, a per-step bf16 rounding would lose them
    assert out[0].item() == torch.tensor(1.0 + 2.0 ** -8).to(torch.bfloat16).item()
    assert out[1].item() == 258.0


# ---------------------------------------------------------------- fp8 emulation (no reference counterpart: parity unpinned)
def test_fp8_activation_quantisation_properties():
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(9, 384, generator=g) * 2).to(torch.bfloat16)
    x[0, :128] = 0
    q, s = O.per_token_group_quant_fp8(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (9, 3)
    assert s[0, 0].item() == pytest.approx(1e-10 / 448.0)
    assert torch.all(q[0, :128].float() == 0)
    # every group uses the whole e4m3 range: its largest magnitude maps to +-448
    assert torch.all(q.float().view(9, 3, 128).abs().amax(-1)[1:] == 448.0)
    deq = q.float().view(9, 3, 128) * s[..., None]
    err = (deq - x.float().view(9, 3, 128)).abs()
    # e4m3 has 3 mantissa bits: relative error <= 2^-4 for normal values, absolute <= scale * 2^-10 for subnormals
    assert torch.all(err <= x.float().view(9, 3, 128).abs() * 2 ** -4 + s[..., None] * 2 ** -9)


def test_fp8_weight_block_quantisation_round_trip():
    g = torch.Generator().manual_seed(1)
    w = (torch.randn(3, 192, 256, generator=g) * 0.02).to(torch.bfloat16)   # 192 rows: a ragged last scale block
    q, s = O.quant_weight_block_fp8(w)
    assert q.shape == w.shape and s.shape == (3, 2, 2)
    deq = O.dequant_weight_block_fp8(q, s)
    assert O.rel_l2(deq, w) <= 4e-2
    # given scales (the benchmark config's recipe) are used as they are
    sc = torch.full((3, 2, 2), 1.0 / 448)
    q2, s2 = O.quant_weight_block_fp8(w, sc)
    assert torch.equal(s2, sc)
    assert O.rel_l2(O.dequant_weight_block_fp8(q2, s2), w) <= 6e-2


def test_fp8_experts_emulation_tracks_bf16_math_on_dequantised_weights():
    g = torch.Generator().manual_seed(2)
    T, H, E, k, I = 48, 256, 4, 2, 128
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.bfloat16)
    q13, s13 = O.quant_weight_block_fp8(w13)
    q2, s2 = O.quant_weight_block_fp8(w2)
    tw, ti, _ = O.fused_topk(x, torch.randn(T, E, generator=g), k, True)
    got = O.fused_experts_fp8(x, q13, s13, q2, s2, tw, ti)
    want = O.fused_experts(x, O.dequant_weight_block_fp8(q13, s13).to(torch.bfloat16),
                           O.dequant_weight_block_fp8(q2, s2).to(torch.bfloat16), tw, ti, "silu", "exact")
    assert O.rel_l2(got, want) <= 8e-2


# ---------------------------------------------------------------- the steps in front of the block
def test_add_rms_norm_oracle_rounding_points():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(6, 256, generator=g).to(torch.bfloat16)
    res = (torch.randn(6, 256, generator=g) * 3).to(torch.bfloat16)
    w = (1 + 0.2 * torch.randn(256, generator=g)).to(torch.bfloat16)
    out, r = O.add_rms_norm(x, res, w, 1e-6)
    # the residual is the bf16 rounding of the fp32 sum; the variance uses the unrounded sum
    s32 = x.float() + res.float()
    assert torch.equal(r, s32.to(torch.bfloat16))
    scale = torch.rsqrt((s32.double() ** 2).mean(-1, keepdim=True) + 1e-6).float()
    want = ((r.float() * scale).to(torch.bfloat16).float() * w.float()).to(torch.bfloat16)
    assert ((out.float() - want.float()).abs() <= want.float().abs() * 2 ** -7 + 1e-6).all()
    # without a residual the input itself is normalised
    out2, r2 = O.add_rms_norm(x, None, w, 1e-6)
    assert torch.equal(r2, x)
    assert out2.shape == x.shape and out2.dtype == torch.bfloat16


def test_router_gate_oracle_is_a_bf16_linear():
    g = torch.Generator().manual_seed(6)
    h = torch.randn(5, 128, generator=g).to(torch.bfloat16)
    wg = (torch.randn(16, 128, generator=g) * 0.02).to(torch.bfloat16)
    lg = O.router_gate(h, wg)
    assert lg.dtype == torch.bfloat16 and lg.shape == (5, 16)
    assert torch.equal(lg, torch.nn.functional.linear(h.float(), wg.float()).to(torch.bfloat16))
