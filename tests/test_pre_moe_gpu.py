"""add_rms_norm / rms_norm and the fused norm + gate projection + top-k call in front of the MoE block."""
import pytest
import torch

from oracle import moe_oracle as O
from oracle.build_ref import load_reference_ops

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


@pytest.fixture(scope="module")
def ref():
    return load_reference_ops()   # None where the compiled reference ops did not travel


def _inputs(T, H, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    res = (torch.randn(T, H, generator=g) * 2).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    return x, res, w


@pytest.mark.parametrize("T,H", [(1, 2048), (64, 2048), (300, 4096), (7, 1024), (5, 256), (3, 6144), (2, 64)])
def test_add_rms_norm_matches_the_reference_kernel_bit_for_bit(ref, T, H):
    from layered_prefill_b200 import ops
    x, res, w = _inputs(T, H, T + H)
    d = _dev()
    xo, ro, wo = x.to(d), res.to(d).clone(), w.to(d)
    out = torch.empty_like(xo)
    ops.add_rms_norm(out, ro, xo, wo, 1e-6)
    want_out, want_res = O.add_rms_norm(x, res, w, 1e-6)
    assert torch.equal(ro.cpu(), want_res), "residual = bf16(x + residual) has no freedom"
    close = (out.cpu().float() - want_out.float()).abs() <= want_out.float().abs() * 2 ** -7 + 1e-6
    assert close.all()
    if ref is not None:
        rr, rout = res.to(d).clone(), torch.empty_like(xo)
        ref.add_rms_norm(rout, rr, xo, wo, 1e-6)
        torch.cuda.synchronize()
        assert torch.equal(rr, ro)
        assert torch.equal(rout, out), "normalised rows differ from the reference kernel"


@pytest.mark.parametrize("T,H", [(64, 2048), (9, 4096), (4, 512)])
def test_rms_norm_matches_the_reference_kernel_and_may_run_in_place(ref, T, H):
    from layered_prefill_b200 import ops
    x, _, w = _inputs(T, H, 3 * T + H)
    d = _dev()
    xo, wo = x.to(d), w.to(d)
    out = torch.empty_like(xo)
    ops.rms_norm(out, xo, wo, 1e-6)
    inplace = xo.clone()
    ops.rms_norm(inplace, inplace, wo, 1e-6)
    assert torch.equal(inplace, out)
    want, _ = O.add_rms_norm(x, None, w, 1e-6)
    assert ((out.cpu().float() - want.float()).abs() <= want.float().abs() * 2 ** -7 + 1e-6).all()
    if ref is not None:
        rout = torch.empty_like(xo)
        ref.rms_norm(rout, xo, wo, 1e-6)
        torch.cuda.synchronize()
        assert torch.equal(rout, out)


@pytest.mark.parametrize("T,H,E,k", [
    (64, 2048, 128, 8),     # decode: the one-kernel path
    (1, 2048, 128, 8),
    (33, 4096, 256, 8),     # 256 experts, two 16-byte groups per lane
    (700, 2048, 128, 8),    # above 512 tokens: norm + tensor-core GEMM + routing kernels
    (40, 512, 64, 4),       # an expert count the one-kernel path does not take
    (2048, 1024, 128, 6),
])
def test_pre_moe_call(ref, T, H, E, k):
    from layered_prefill_b200 import fused_moe, ops
    x, res, w = _inputs(T, H, T + E)
    g = torch.Generator().manual_seed(99)
    wg = (torch.randn(E, H, generator=g) * 0.02).to(torch.bfloat16)
    d = _dev()
    xo, ro, wo, wgo = x.to(d), res.to(d).clone(), w.to(d), wg.to(d)
    normed, r2, tw, ti, logits = fused_moe.pre_moe(xo, ro, wo, 1e-6, wgo, k, True, return_logits=True)
    assert ops.read_status(d) == 0
    assert r2.data_ptr() == ro.data_ptr()
    # norm: same bits as the stand-alone op (which is pinned against the reference kernel above)
    r_op, out_op = res.to(d).clone(), torch.empty_like(xo)
    ops.add_rms_norm(out_op, r_op, xo, wo, 1e-6)
    assert torch.equal(r_op, ro) and torch.equal(out_op, normed)
    # gate projection: bf16 rounding of an fp32 product; the summation order is free, so one bf16 ulp of slack
    want_logits = O.router_gate(normed.cpu(), wg)
    diff = (logits.cpu().float() - want_logits.float()).abs()
    assert (diff <= want_logits.float().abs() * 2 ** -7 + 2e-3).all(), diff.max()
    # routing: exactly the routing kernel's answer on these logits
    otw, oti, _ = O.fused_topk(normed.cpu(), logits.cpu(), k, True)
    assert torch.equal(ti.cpu(), oti)
    assert torch.allclose(tw.cpu(), otw, rtol=1e-6, atol=1e-8)
    # and the call without the optional logits output gives the same routing
    ro2 = res.to(d).clone()
    n2, _, tw2, ti2 = fused_moe.pre_moe(xo, ro2, wo, 1e-6, wgo, k, True)
    assert torch.equal(n2, normed) and torch.equal(ti2, ti) and torch.equal(tw2, tw)
