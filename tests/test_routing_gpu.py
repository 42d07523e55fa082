"""Router and permutation kernels against the CPU oracle (bit-exact ids) through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _route_gpu(logits, k, renorm):
    from layered_prefill_b200 import fused_moe
    x = torch.empty(logits.shape[0], 8, device=_dev())
    return fused_moe.fused_topk(x, logits.to(_dev()), k, renorm)


@pytest.mark.parametrize("E", [1, 2, 4, 8, 16, 32, 64, 128, 256])
@pytest.mark.parametrize("T", [1, 3, 17, 130])
def test_topk_pow2_bit_exact_ids(E, T):
    g = torch.Generator().manual_seed(E * 1000 + T)
    k = min(8, E)
    logits = torch.randn(T, E, generator=g)
    for renorm in (False, True):
        w, ids, tei = _route_gpu(logits, k, renorm)
        ow, oids, otei = O.topk_softmax(logits, k, renorm)
        assert torch.equal(ids.cpu(), oids), f"E={E} T={T}"
        assert torch.equal(tei.cpu(), otei)
        np.testing.assert_allclose(w.cpu().numpy(), ow.numpy(), rtol=1e-6, atol=1e-8)


def test_topk_bf16_logits_equal_fp32_upcast():
    g = torch.Generator().manual_seed(7)
    logits = torch.randn(257, 128, generator=g).to(torch.bfloat16)
    w1, i1, _ = _route_gpu(logits, 8, True)
    w2, i2, _ = _route_gpu(logits.float(), 8, True)
    assert torch.equal(i1, i2) and torch.equal(w1, w2)
    ow, oi, _ = O.topk_softmax(logits, 8, True)
    assert torch.equal(i1.cpu(), oi)
    # bf16 logits collide often: this is the tie-breaking case
    assert (logits.float().sort(dim=-1).values.diff(dim=-1) == 0).any()


def test_topk_exact_ties_lowest_index_wins():
    logits = torch.zeros(5, 128)
    logits[1, 40:50] = 3.0
    logits[2, [127, 0, 64]] = 1.0
    logits[3] = torch.arange(128).float().flip(0) * 0  # all equal
    logits[4, 100:] = 2.0
    _, ids, _ = _route_gpu(logits, 8, True)
    _, oids, _ = O.topk_softmax(logits, 8, True)
    assert torch.equal(ids.cpu(), oids)
    assert ids[0].tolist() == list(range(8))
    assert ids[1].tolist() == list(range(40, 48))
    assert ids[2].tolist()[:3] == [0, 64, 127]


@pytest.mark.parametrize("E", [3, 96, 160, 384])
def test_topk_generic_expert_counts(E):
    g = torch.Generator().manual_seed(E)
    logits = torch.randn(33, E, generator=g)
    k = min(4, E)
    w, ids, _ = _route_gpu(logits, k, False)
    ow, oids, _ = O.topk_softmax(logits, k, False)
    assert torch.equal(ids.cpu(), oids)
    np.testing.assert_allclose(w.cpu().numpy(), ow.numpy(), rtol=2e-6, atol=1e-8)


def test_topk_ops_signature_and_full_size():
    """ops.topk_softmax(topk_weights, topk_indices, token_expert_indices, gating_output) at T=8192, E=128."""
    from layered_prefill_b200 import ops
    g = torch.Generator().manual_seed(11)
    logits = (torch.randn(8192, 128, generator=g) + torch.randn(128, generator=g)).to(torch.bfloat16).float()
    d = _dev()
    w = torch.empty(8192, 8, device=d)
    ids = torch.empty(8192, 8, dtype=torch.int32, device=d)
    tei = torch.empty(8192, 8, dtype=torch.int32, device=d)
    ops.topk_softmax(w, ids, tei, logits.to(d))
    ow, oids, otei = O.topk_softmax(logits, 8, False)
    assert torch.equal(ids.cpu(), oids) and torch.equal(tei.cpu(), otei)
    np.testing.assert_allclose(w.cpu().numpy(), ow.numpy(), rtol=1e-6, atol=1e-9)
    # every row: k distinct experts
    assert (ids.sort(dim=-1).values.diff(dim=-1) > 0).all()


def _align_gpu(ids, bs, E):
    from layered_prefill_b200 import fused_moe
    return fused_moe.moe_align_block_size(ids.to(_dev()), bs, E)


@pytest.mark.parametrize("T,k,E,bs", [
    (1, 1, 1, 1), (3, 2, 4, 4), (17, 2, 8, 16), (64, 8, 128, 16), (64, 8, 128, 128), (256, 8, 128, 64),
    (512, 8, 128, 64), (513, 8, 128, 64), (8192, 8, 128, 64), (8192, 8, 128, 128), (1000, 6, 60, 32),
    (40000, 2, 1024, 8),
])
def test_align_bit_exact(T, k, E, bs):
    g = torch.Generator().manual_seed(T + 7 * E + bs)
    # skewed expert popularity, distinct experts per token
    pop = torch.rand(E, generator=g) ** 3 + 1e-3
    ids = torch.multinomial(pop.expand(T, E), k, replacement=False, generator=g).to(torch.int32)
    s, e, post = _align_gpu(ids, bs, E)
    os_, oe, opost = O.moe_align_block_size(ids, bs, E)
    assert int(post.cpu()) == int(opost)
    assert torch.equal(e.cpu(), oe)
    assert torch.equal(s.cpu(), os_)  # the kernel emits the canonical ascending order itself
    c = O.canonicalize_sorted_ids(s.cpu(), e.cpu(), int(post.cpu()), bs, T * k)
    assert torch.equal(c, os_)


def test_align_edge_cases():
    # empty input
    s, e, post = _align_gpu(torch.zeros(0, 8, dtype=torch.int32), 16, 128)
    assert int(post.cpu()) == 0 and (e.cpu() == 0).all() and (s.cpu() == 0).all()
    # one expert takes everything; ids outside [0,E) are skipped
    ids = torch.full((300, 2), 5, dtype=torch.int32)
    ids[:, 1] = 9
    ids[7, 0] = 200
    s, e, post = _align_gpu(ids, 64, 16)
    os_, oe, opost = O.moe_align_block_size(ids, 64, 16)
    assert int(post.cpu()) == int(opost) and torch.equal(s.cpu(), os_) and torch.equal(e.cpu(), oe)
    # exactly block_size tokens for an expert: no padding block
    ids = torch.zeros(64, 1, dtype=torch.int32)
    s, e, post = _align_gpu(ids, 64, 4)
    assert int(post.cpu()) == 64 and s.cpu()[:64].tolist() == list(range(64))


def test_align_is_deterministic_run_to_run():
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 128, (8192, 8), generator=g).to(torch.int32)
    a = _align_gpu(ids, 64, 128)
    b = _align_gpu(ids, 64, 128)
    assert all(torch.equal(x, y) for x, y in zip(a, b))


def test_elementwise_ops_match_oracle():
    from layered_prefill_b200 import ops
    g = torch.Generator().manual_seed(9)
    d = _dev()
    x = (torch.randn(77, 2 * 768, generator=g) * 3).to(torch.bfloat16)
    out = torch.empty(77, 768, dtype=torch.bfloat16, device=d)
    ops.silu_and_mul(out, x.to(d))
    want = O.silu_and_mul(x)
    assert (out.cpu().float() - want.float()).abs().max() <= 2 ** -7 * want.float().abs().max()
    assert (out.cpu() != want).float().mean() < 1e-3  # expf may differ in the last bit before rounding
    out2 = torch.empty(77, 768, dtype=torch.bfloat16, device=d)
    ops.swigluoai_and_mul(out2, x.to(d), 1.702, 7.0)
    want2 = O.swigluoai_and_mul(x)
    assert (out2.cpu() != want2).float().mean() < 1e-3
    c3 = torch.randn(50, 8, 2048, generator=g).to(torch.bfloat16)
    o = torch.empty(50, 2048, dtype=torch.bfloat16, device=d)
    ops.moe_sum(c3.to(d), o)
    assert torch.equal(o.cpu(), O.moe_sum(c3))
