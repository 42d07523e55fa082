"""This library next to the reference's OWN fused MoE path on the same seeded tensors: its `fused_topk` (CUDA op)
and `fused_experts` (Triton `fused_moe_kernel` twice + its activation op + `moe_sum`,
nanovllm/layers/for_moe/fused_moe.py:393-633), its `FusedMoE` layer (nanovllm/layers/fused_moe.py:218-787) and its
`Qwen3MoeSparseMoeBlock` (nanovllm/models/qwen3_moe.py:66-116), all imported unmodified from the staged copy under
oracle/_ref/ (made by oracle/build_ref.py where the reference tree is mounted; the tests skip where it is absent).

Three comparisons per case:
  * ours vs the reference: `topk_ids` equal, outputs within max-abs 2e-2 and relative L2 5e-3 (bf16);
  * the CPU oracle vs the reference, same bounds: this is what pins the oracle's GEMM leg;
  * the reference's caller (layer / sparse block) with this library's functions patched into its namespace.
"""
import os

import pytest
import torch

from oracle import moe_oracle as O
from oracle.build_ref import load_reference_package

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-2
REL_L2 = 5e-3


@pytest.fixture(scope="module")
def ref():
    pkg = load_reference_package()
    if pkg is None:
        pytest.skip("oracle/_ref/nanovllm not staged (needs the reference tree at build time)")
    import nanovllm.layers.for_moe.fused_moe as rfm
    return rfm


@pytest.fixture(scope="module")
def single_rank_group():
    """The reference's layers read torch.distributed's world size in their constructors."""
    import torch.distributed as dist
    created = False
    if not dist.is_initialized():
        import socket
        with socket.socket() as sock:  # any free port: the group has one member, nobody else needs to know it
            sock.bind(("127.0.0.1", 0))
            port = sock.getsockname()[1]
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
        created = True
    yield
    if created:
        dist.destroy_process_group()


def _dev():
    return torch.device("cuda", 0)


def _bounds(got, want, what, scaled=False):
    """max-abs <= 2e-2 and relative L2 <= 5e-3. scaled=True (the synthetic variants below, whose outputs reach
    magnitudes of 4 to 30 where one bf16 ulp alone exceeds 2e-2) allows two bf16 ulps of the largest output."""
    ma, rl = O.max_abs(got, want), O.rel_l2(got, want)
    bound = max(MAX_ABS, 2 ** -7 * float(want.float().abs().max())) if scaled else MAX_ABS
    assert rl <= REL_L2 and ma <= bound, f"{what}: rel-L2 {rl:.3e}, max-abs {ma:.3e} (bound {bound:.3e})"
    return ma, rl


def _reference_block(rfm, x, logits, w13, w2, k, activation="silu", b13=None, b2=None):
    tw, ti, _ = rfm.fused_topk(x, logits, k, True)
    out = rfm.fused_experts(x.clone(), w13, w2, b13, b2, tw, ti, inplace=True, activation=activation)
    return tw, ti, out


@pytest.mark.parametrize("name", ["qwen3-30b-a3b-t256", "qwen3-30b-a3b-decode-t64", "qwen3-30b-a3b-prefill-t8192"])
def test_block_against_reference_on_benchmark_configs(ref, name):
    from layered_prefill_b200 import fused_moe, ops, workload
    wl = workload.WORKLOADS[name]
    inp = workload.make_inputs(wl, seed=0)
    d = _dev()
    x, lg, w13, w2 = (inp[n].to(d) for n in ("x", "router_logits", "w13", "w2"))
    rtw, rti, rout = _reference_block(ref, x, lg, w13, w2, wl.top_k)
    otw, oti, _ = fused_moe.fused_topk(x, lg, wl.top_k, True)
    got = fused_moe.fused_experts(x.clone(), w13, w2, None, None, otw, oti, inplace=True)
    torch.cuda.synchronize()
    assert ops.read_status(d) == 0
    assert torch.equal(rti, oti), "topk_ids differ from the reference's"
    assert torch.allclose(rtw, otw, rtol=1e-6, atol=1e-8)
    _bounds(got.cpu(), rout.cpu(), f"{name}: ours vs reference")
    # the one-call block too (router + experts behind one C entry)
    blk = fused_moe.fused_moe_forward(x, lg, w13, w2, wl.top_k, True, inplace=False)
    _bounds(blk.cpu(), rout.cpu(), f"{name}: fused_moe_forward vs reference")
    # the CPU oracle against the reference: every token up to 256, a spread sample beyond
    idx = torch.arange(wl.T) if wl.T <= 256 else torch.arange(0, wl.T, wl.T // 96)[:96]
    want = O.fused_experts(inp["x"][idx], inp["w13"], inp["w2"], rtw.cpu()[idx], rti.cpu()[idx])
    _bounds(want, rout.cpu()[idx], f"{name}: oracle vs reference")
    ctw, cti, _ = O.fused_topk(inp["x"], inp["router_logits"], wl.top_k, True)
    assert torch.equal(cti, rti.cpu()), "oracle routing differs from the reference's"


@pytest.mark.parametrize("T,H,E,k,I,activation,bias", [
    (300, 512, 16, 4, 128, "swigluoai", True),    # gpt-oss form: interleaved gate/up, clamp, expert biases
    (64, 2048, 128, 8, 96, "silu", False),        # one rank's shapes of config 2 at TP=8 (I/tp = 96)
    (512, 1024, 32, 2, 192, "silu", True),        # biases with the plain activation, I/tp = 192
    (1, 256, 8, 2, 64, "silu", False),            # a single token
])
def test_variants_against_reference(ref, T, H, E, k, I, activation, bias):
    from layered_prefill_b200 import fused_moe, ops
    g = torch.Generator().manual_seed(T * 7 + I)
    scale = 0.1 if activation == "swigluoai" else 0.05
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * scale).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * scale).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g).to(torch.bfloat16)
    b13 = (torch.randn(E, 2 * I, generator=g) * 0.1).to(torch.bfloat16) if bias else None
    b2 = (torch.randn(E, H, generator=g) * 0.1).to(torch.bfloat16) if bias else None
    d = _dev()
    xd, lgd, w13d, w2d = x.to(d), logits.to(d), w13.to(d), w2.to(d)
    b13d, b2d = (b13.to(d), b2.to(d)) if bias else (None, None)
    rtw, rti, rout = _reference_block(ref, xd, lgd, w13d, w2d, k, activation, b13d, b2d)
    otw, oti, _ = fused_moe.fused_topk(xd, lgd, k, True)
    assert torch.equal(rti, oti)
    got = fused_moe.fused_experts(xd, w13d, w2d, b13d, b2d, otw, oti, inplace=False, activation=activation)
    torch.cuda.synchronize()
    assert ops.read_status(d) == 0
    _bounds(got.cpu(), rout.cpu(), "ours vs reference", scaled=True)
    want = O.fused_experts(x, w13, w2, rtw.cpu(), rti.cpu(), activation, "ref_rounding", b13, b2)
    _bounds(want, rout.cpu(), "oracle vs reference", scaled=True)


def _fill_through_loaders(layers, E, I, H, bias, seed, fused=False):
    """Checkpoint-shaped tensors pushed through every layer's own weight_loader, as utils/loader.py:37-93 calls it:
    per expert gate / up / down (Qwen3-MoE), or all-expert fused tensors and biases (gpt-oss, fused=True)."""
    g = torch.Generator().manual_seed(seed)
    if fused:
        gate_up = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16)
        down = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.bfloat16)
        for m in layers:
            dev = m.w13_weight.device
            m.weight_loader(m.w13_weight, gate_up.to(dev), "model.layers.0.mlp.experts.gate_up_proj_blocks", "w13", 0)
            m.weight_loader(m.w2_weight, down.to(dev), "model.layers.0.mlp.experts.down_proj_blocks", "w2", 0)
    else:
        for e in range(E):
            gate = (torch.randn(I, H, generator=g) * 0.05).to(torch.bfloat16)
            up = (torch.randn(I, H, generator=g) * 0.05).to(torch.bfloat16)
            down = (torch.randn(H, I, generator=g) * 0.05).to(torch.bfloat16)
            for m in layers:
                dev = m.w13_weight.device
                m.weight_loader(m.w13_weight, gate.to(dev), "experts.w13_weight", "w1", e)
                m.weight_loader(m.w13_weight, up.to(dev), "experts.w13_weight", "w3", e)
                m.weight_loader(m.w2_weight, down.to(dev), "experts.w2_weight", "w2", e)
    if bias:
        b13 = (torch.randn(E, 2 * I, generator=g) * 0.1).to(torch.bfloat16)
        b2 = (torch.randn(E, H, generator=g) * 0.1).to(torch.bfloat16)
        for m in layers:
            dev = m.w13_weight.device
            m.weight_loader(m.w13_bias, b13.to(dev), "model.layers.0.mlp.experts.gate_up_proj_bias", "w13", 0)
            m.weight_loader(m.w2_bias, b2.to(dev), "model.layers.0.mlp.experts.down_proj_bias", "w2", 0)


@pytest.mark.parametrize("activation,bias", [("silu", False), ("swigluoai", True)])
def test_fused_moe_layer_against_reference_layer(ref, single_rank_group, activation, bias):
    """Both FusedMoE modules, same constructor arguments, weights through both weight_loaders, same forward."""
    import nanovllm.layers.fused_moe as rlayer
    from layered_prefill_b200 import layer as olayer, ops
    T, H, E, k, I = 200, 512, 16, 4, 128
    d = _dev()
    kw = dict(num_experts=E, top_k=k, hidden_size=H, intermediate_size=I, params_dtype=torch.bfloat16,
              reduce_results=False, renormalize=True, activation=activation, has_bias=bias)
    with torch.device(d):
        rm, om = rlayer.FusedMoE(**kw), olayer.FusedMoE(**kw)
    _fill_through_loaders([rm, om], E, I, H, bias, seed=5, fused=activation == "swigluoai")
    assert torch.equal(rm.w13_weight, om.w13_weight) and torch.equal(rm.w2_weight, om.w2_weight)
    if bias:
        assert torch.equal(rm.w13_bias, om.w13_bias) and torch.equal(rm.w2_bias, om.w2_bias)
    g = torch.Generator().manual_seed(9)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(d)
    lg = torch.randn(T, E, generator=g).to(torch.bfloat16).to(d)
    xr, xo = x.clone(), x.clone()
    rout = rm(hidden_states=xr, router_logits=lg)
    oout = om(hidden_states=xo, router_logits=lg)
    torch.cuda.synchronize()
    assert ops.read_status(d) == 0
    assert oout.data_ptr() == xo.data_ptr() and rout.data_ptr() == xr.data_ptr()  # both overwrite their input
    _bounds(oout.cpu(), rout.cpu(), "FusedMoE.forward vs the reference's", scaled=True)
    # and the CPU oracle on the loaded weights
    b13 = om.w13_bias.cpu() if bias else None
    b2 = om.w2_bias.cpu() if bias else None
    tw, ti, _ = O.fused_topk(x.cpu(), lg.cpu(), k, True)
    want = O.fused_experts(x.cpu(), om.w13_weight.cpu(), om.w2_weight.cpu(), tw, ti, activation, "ref_rounding", b13, b2)
    _bounds(oout.cpu(), want, "FusedMoE.forward vs oracle", scaled=True)


def test_library_patched_into_the_reference_sparse_moe_block(ref, single_rank_group, monkeypatch):
    """The reference's own Qwen3MoeSparseMoeBlock.forward (gate linear -> FusedMoE -> reduce) run twice: as it is,
    and with this library's fused_topk / fused_experts / tensor_model_parallel_all_reduce patched into the
    reference modules' namespaces. Same weights, same tokens: the patched block must match the stock one."""
    import nanovllm.layers.fused_moe as rlayer
    import nanovllm.models.qwen3_moe as rmodel
    from transformers import Qwen3MoeConfig
    from layered_prefill_b200 import custom_all_reduce as ocar, fused_moe as ofm, ops
    cfg = Qwen3MoeConfig(hidden_size=1024, num_experts=32, num_experts_per_tok=4, moe_intermediate_size=256,
                         norm_topk_prob=True)
    d = _dev()
    torch.manual_seed(0)
    saved = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(d):
            stock = rmodel.Qwen3MoeSparseMoeBlock(cfg)
    finally:
        torch.set_default_dtype(saved)
    E, I, H = cfg.num_experts, cfg.moe_intermediate_size, cfg.hidden_size
    _fill_through_loaders([stock.experts], E, I, H, False, seed=13)
    g = torch.Generator().manual_seed(14)
    stock.gate.weight.data.copy_((torch.randn(E, H, generator=g) * 0.02).to(torch.bfloat16))
    for T in (64, 1536):
        x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(d)
        want = stock(x.clone())
        with monkeypatch.context() as m:
            m.setattr(ref, "fused_topk", ofm.fused_topk)
            m.setattr(stock.experts.quant_method, "fused_experts", ofm.fused_experts)
            m.setattr(rlayer, "tensor_model_parallel_all_reduce", ocar.tensor_model_parallel_all_reduce)
            launches0 = ops.launch_count()
            got = stock(x.clone())
            assert ops.launch_count() - launches0 >= 4, "the patched block did not run this library's kernels"
        torch.cuda.synchronize()
        assert ops.read_status(d) == 0
        _bounds(got.cpu(), want.cpu(), f"patched sparse MoE block, T={T}", scaled=True)


def test_reference_safetensors_loader_fills_this_librarys_layers(ref, single_rank_group, tmp_path):
    """The reference's own checkpoint loader (nanovllm/utils/loader.py:37-116: name pattern -> parameter, shard id and
    expert id -> `moe_layer.weight_loader(...)`; every other tensor through its parameter's `weight_loader`) driven
    over a synthetic Qwen3-MoE-named safetensors file into a module tree built from THIS library's FusedMoE and
    RowParallelLinear: the loaded parameters must be the checkpoint's tensors in the reference's layout."""
    import nanovllm.utils.loader as rloader
    from safetensors.torch import save_file
    from torch import nn
    from layered_prefill_b200.layer import FusedMoE
    from layered_prefill_b200.linear import RowParallelLinear
    E, k, H, I, L = 4, 2, 64, 32, 2

    class Mlp(nn.Module):
        def __init__(self):
            super().__init__()
            self.experts = FusedMoE(E, k, H, I, params_dtype=torch.bfloat16)
            self.gate = nn.Linear(H, E, bias=False, dtype=torch.bfloat16)

    class Attn(nn.Module):
        def __init__(self):
            super().__init__()
            self.o_proj = RowParallelLinear(H, H).to(torch.bfloat16)

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.mlp, self.self_attn = Mlp(), Attn()

    class Inner(nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = nn.ModuleList([Layer() for _ in range(L)])

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.model = Inner()

    model = Model()
    g = torch.Generator().manual_seed(77)
    ckpt = {}
    for li in range(L):
        for e in range(E):
            for proj, shape in (("gate_proj", (I, H)), ("up_proj", (I, H)), ("down_proj", (H, I))):
                ckpt[f"model.layers.{li}.mlp.experts.{e}.{proj}.weight"] = torch.randn(*shape, generator=g).to(torch.bfloat16)
        ckpt[f"model.layers.{li}.mlp.gate.weight"] = torch.randn(E, H, generator=g).to(torch.bfloat16)
        ckpt[f"model.layers.{li}.self_attn.o_proj.weight"] = torch.randn(H, H, generator=g).to(torch.bfloat16)
    save_file(ckpt, str(tmp_path / "model.safetensors"))
    saved = rloader.FusedMoE
    rloader.FusedMoE = FusedMoE  # the loader finds MoE layers by isinstance
    try:
        rloader.load_model(model, str(tmp_path))
    finally:
        rloader.FusedMoE = saved
    for li in range(L):
        layer = model.model.layers[li]
        for e in range(E):
            pre = f"model.layers.{li}.mlp.experts.{e}."
            assert torch.equal(layer.mlp.experts.w13_weight[e, :I], ckpt[pre + "gate_proj.weight"])
            assert torch.equal(layer.mlp.experts.w13_weight[e, I:], ckpt[pre + "up_proj.weight"])
            assert torch.equal(layer.mlp.experts.w2_weight[e], ckpt[pre + "down_proj.weight"])
        assert torch.equal(layer.mlp.gate.weight, ckpt[f"model.layers.{li}.mlp.gate.weight"])
        assert torch.equal(layer.self_attn.o_proj.weight, ckpt[f"model.layers.{li}.self_attn.o_proj.weight"])
