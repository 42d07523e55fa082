"""Our ops next to the reference's own CUDA ops, compiled from the reference's sources into
oracle/_ref/ (a checker that travels as a binary; skipped where it was not built)."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from oracle.build_ref import load_reference_ops

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    mod = load_reference_ops()
    if mod is None:
        pytest.skip("oracle/_ref/nanovllm_ref_ops.so not built (needs the reference tree at build time)")
    return mod


def _dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("T,E,k", [(64, 128, 8), (8192, 128, 8), (257, 64, 4), (33, 256, 8), (100, 8, 2), (77, 96, 4)])
def test_topk_softmax_against_reference_kernel(ref, T, E, k):
    from layered_prefill_b200 import ops
    g = torch.Generator().manual_seed(T + E)
    logits = (torch.randn(T, E, generator=g) + torch.randn(E, generator=g)).to(torch.bfloat16).float().to(_dev())
    outs = []
    for fn in (ref.topk_softmax, ops.topk_softmax):
        w = torch.empty(T, k, device=_dev())
        ids = torch.empty(T, k, dtype=torch.int32, device=_dev())
        tei = torch.empty(T, k, dtype=torch.int32, device=_dev())
        fn(w, ids, tei, logits)
        outs.append((w, ids, tei))
    torch.cuda.synchronize()
    (rw, ri, rt), (ow, oi, ot) = outs
    assert torch.equal(ri, oi), "topk_ids differ from the reference kernel"
    assert torch.equal(rt, ot)
    pow2 = E & (E - 1) == 0
    if pow2:
        assert torch.equal(rw, ow), "same arithmetic order: weights must be bit-identical"
    else:
        np.testing.assert_allclose(ow.cpu().numpy(), rw.cpu().numpy(), rtol=2e-6, atol=1e-9)
    # and the CPU oracle agrees with both on the ids
    _, cpu_ids, _ = O.topk_softmax(logits.cpu(), k, False)
    assert torch.equal(cpu_ids, oi.cpu())


@pytest.mark.parametrize("T,k,E,bs", [(64, 8, 128, 16), (256, 8, 128, 64), (8192, 8, 128, 64), (1000, 6, 60, 32)])
def test_moe_align_block_size_against_reference_kernel(ref, T, k, E, bs):
    from layered_prefill_b200 import ops
    g = torch.Generator().manual_seed(T * 3 + bs)
    pop = torch.rand(E, generator=g) ** 3 + 1e-3
    ids = torch.multinomial(pop.expand(T, E), k, replacement=False, generator=g).to(torch.int32).to(_dev())
    numel = T * k
    cap = numel + E * (bs - 1)
    outs = []
    for fn in (ref.moe_align_block_size, ops.moe_align_block_size):
        s = torch.empty(cap, dtype=torch.int32, device=_dev())
        s.fill_(numel)  # the reference's Python wrapper does this (for_moe/fused_moe.py:61)
        e = torch.empty(-(-cap // bs), dtype=torch.int32, device=_dev())
        p = torch.empty(1, dtype=torch.int32, device=_dev())
        fn(ids, E, bs, s, e, p)
        outs.append((s, e, p))
    torch.cuda.synchronize()
    (rs, re_, rp), (os_, oe, op) = outs
    post = int(rp.cpu())
    assert post == int(op.cpu())
    nblk = post // bs
    assert torch.equal(re_[:nblk], oe[:nblk]), "expert_ids differ from the reference kernel"
    assert torch.equal(re_.cpu(), oe.cpu())
    canon = O.canonicalize_sorted_ids(rs.cpu(), re_.cpu(), post, bs, numel)
    assert torch.equal(canon, os_.cpu()), "sorted_token_ids differ after canonical ordering"


def test_silu_and_mul_against_reference_kernel(ref):
    from layered_prefill_b200 import ops
    g = torch.Generator().manual_seed(4)
    x = (torch.randn(300, 2 * 768, generator=g) * 3).to(torch.bfloat16).to(_dev())
    a = torch.empty(300, 768, dtype=torch.bfloat16, device=_dev())
    b = torch.empty_like(a)
    ref.silu_and_mul(a, x)
    ops.silu_and_mul(b, x)
    torch.cuda.synchronize()
    assert torch.equal(a, b), "same expf, same roundings: bit-identical"
    c, d = torch.empty_like(a), torch.empty_like(a)
    ref.swigluoai_and_mul(c, x, 1.702, 7.0)
    ops.swigluoai_and_mul(d, x, 1.702, 7.0)
    torch.cuda.synchronize()
    assert torch.equal(c, d)
