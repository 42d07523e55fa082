"""Host-side mirror of nanovllm/layers/for_moe/fused_moe.py: `fused_topk`, `moe_align_block_size`,
`fused_experts` / `fused_experts_impl` with the reference's signatures, backed by libmoe_b200.

What is different underneath: one C call runs permutation, both grouped tcgen05 GEMMs (activation
and routed-weight scaling in their epilogues) and the k-slot sum on the current stream; the tile
shape is chosen inside the library from the shapes, so there is no Triton config lookup
(for_moe/fused_moe.py:318-390 has no counterpart here). Quantised paths are rejected, as they are
by the reference's asserts (for_moe/fused_moe.py:248-249,571,607).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import ops
from ._lib import ACT_CODES, check, lib


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def fused_topk(hidden_states: torch.Tensor, gating_output: torch.Tensor, topk: int, renormalize: bool):
    """for_moe/fused_moe.py:393-419. Returns (topk_weights f32 [M,k], topk_ids i32 [M,k],
    token_expert_indices i32 [M,k]). bf16 logits are consumed directly (the upcast is exact) and the
    renormalisation is applied by the same kernel."""
    assert hidden_states.shape[0] == gating_output.shape[0], "Number of tokens mismatch"
    M = hidden_states.shape[0]
    dev = hidden_states.device
    topk_weights = torch.empty(M, topk, dtype=torch.float32, device=dev)
    topk_ids = torch.empty(M, topk, dtype=torch.int32, device=dev)
    token_expert_indices = torch.empty(M, topk, dtype=torch.int32, device=dev)
    g = gating_output if gating_output.dtype in (torch.float32, torch.bfloat16) else gating_output.float()
    g = g.contiguous()
    E = g.size(-1)
    with torch.cuda.device(dev):
        check(lib.moe_b200_topk_softmax(g.data_ptr(), int(g.dtype == torch.bfloat16), topk_weights.data_ptr(),
                                        topk_ids.data_ptr(), token_expert_indices.data_ptr(), M, E, topk,
                                        int(bool(renormalize)), torch.cuda.current_stream().cuda_stream))
    return topk_weights, topk_ids, token_expert_indices


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int
                         ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """for_moe/fused_moe.py:17-70: same buffer sizes and fill value; ids inside an expert come out in
    ascending order (the reference leaves that order to atomic arrival)."""
    max_num_tokens_padded = topk_ids.numel() + num_experts * (block_size - 1)
    sorted_ids = torch.empty((max_num_tokens_padded,), dtype=torch.int32, device=topk_ids.device)
    max_num_m_blocks = cdiv(max_num_tokens_padded, block_size)
    expert_ids = torch.empty((max_num_m_blocks,), dtype=torch.int32, device=topk_ids.device)
    num_tokens_post_pad = torch.empty((1), dtype=torch.int32, device=topk_ids.device)
    ops.moe_align_block_size(topk_ids, num_experts, block_size, sorted_ids, expert_ids, num_tokens_post_pad)
    return sorted_ids, expert_ids, num_tokens_post_pad


class _Workspaces:
    """One scratch tensor per device, reused across calls (no per-call malloc). It grows when a larger request
    comes; outgrown tensors are kept alive, because a CUDA graph captured earlier still holds their address.
    Growing inside a stream capture is refused (the new tensor would belong to the capture's private pool):
    call `reserve_workspace` for the largest batch before capturing. All streams of a device share the buffer,
    so calls on different streams must be ordered by the caller."""

    def __init__(self) -> None:
        self._buf: dict[int, torch.Tensor] = {}
        self._outgrown: list[torch.Tensor] = []

    def get(self, device: torch.device, nbytes: int) -> torch.Tensor:
        idx = device.index if device.index is not None else torch.cuda.current_device()
        cur = self._buf.get(idx)
        if cur is None or cur.numel() < nbytes:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError(
                    f"the MoE workspace would have to grow to {nbytes} bytes inside a CUDA-graph capture; "
                    "call fused_moe.reserve_workspace(...) for the largest batch before capturing")
            if cur is not None:
                self._outgrown.append(cur)
            cur = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=torch.device("cuda", idx))
            self._buf[idx] = cur
        return cur


_workspaces = _Workspaces()


def reserve_workspace(device: torch.device, max_tokens: int, num_experts: int, top_k: int, hidden_size: int,
                      intermediate_size_per_partition: int, fp8: bool = False) -> int:
    """Sizes the device's scratch buffer for batches of up to `max_tokens` tokens, so that later calls (inside
    CUDA-graph captures too) never allocate. Returns the size in bytes."""
    args = (int(max_tokens), int(num_experts), int(top_k), int(hidden_size), int(intermediate_size_per_partition))
    nbytes = max(lib.moe_b200_fused_moe_workspace_bytes(*args),
                 lib.moe_b200_fused_experts_fp8_workspace_bytes(*args) if fp8 else 0)
    _workspaces.get(device, nbytes)
    return int(nbytes)


def _check_experts_args(hidden_states, w1, w2, topk_weights, topk_ids, activation, **quant):
    assert hidden_states.size(1) == w1.size(2), f"Hidden size mismatch {hidden_states.size(1)} != {w1.size(2)}"
    assert topk_weights.size() == topk_ids.size(), "topk shape mismatch"
    assert hidden_states.is_contiguous(), "Hidden_states must be contiguous"
    assert w1.stride(-1) == 1, "Stride of last dimension must be 1"
    assert w2.stride(-1) == 1, "Stride of last dimension must be 1"
    if hidden_states.dtype != torch.bfloat16 or w1.dtype != torch.bfloat16 or w2.dtype != torch.bfloat16:
        raise ValueError(f"Unsupported compute_type: {hidden_states.dtype} (this build computes in bfloat16)")
    if activation not in ACT_CODES:
        raise ValueError(f"Unsupported FusedMoe activation: {activation}")
    for name, v in quant.items():
        assert v is None, f"{name} is not supported (the reference asserts the same)"
    if not hidden_states.is_cuda:
        raise RuntimeError("fused_experts needs CUDA tensors; there is no CPU path")
    assert w1.is_contiguous() and w2.is_contiguous(), "expert weights must be contiguous [E, 2I, H] / [E, H, I]"


def fused_experts_impl(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor,
                       topk_ids: torch.Tensor, inplace: bool = False, activation: str = "silu",
                       apply_router_weight_on_input: bool = False, per_channel_quant: bool = False,
                       global_num_experts: int = -1, expert_map: Optional[torch.Tensor] = None,
                       w1_scale=None, w2_scale=None, w1_zp=None, w2_zp=None, a1_scale=None, a2_scale=None,
                       block_shape=None, w1_bias: Optional[torch.Tensor] = None,
                       w2_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """for_moe/fused_moe.py:461-633. With e4m3 weights, `w1_scale` / `w2_scale` and `block_shape=[128, 128]` (arguments
    the reference declares and asserts unused) the block-scaled fp8 path runs instead."""
    if w1.dtype in (torch.float8_e4m3fn, torch.uint8):
        return _fused_experts_fp8(hidden_states, w1, w2, topk_weights, topk_ids, inplace, activation, w1_scale,
                                  w2_scale, block_shape, w1_bias, w2_bias, a1_scale, a2_scale, w1_zp, w2_zp,
                                  expert_map, apply_router_weight_on_input)
    _check_experts_args(hidden_states, w1, w2, topk_weights, topk_ids, activation, w1_scale=w1_scale,
                        w2_scale=w2_scale, w1_zp=w1_zp, w2_zp=w2_zp, a1_scale=a1_scale, a2_scale=a2_scale,
                        block_shape=block_shape, expert_map=expert_map)
    if apply_router_weight_on_input:
        raise NotImplementedError("apply_router_weight_on_input=True is not used by the reference's models")
    T, H = hidden_states.shape
    E, two_i, _ = w1.shape
    inter = two_i // 2
    assert w2.shape == (E, H, inter), f"w2 shape {tuple(w2.shape)} does not match w13 {tuple(w1.shape)}"
    if global_num_experts not in (-1, E):
        raise NotImplementedError("expert parallelism (global_num_experts != local) is not part of the reference's path")
    k = topk_ids.size(1)
    out = hidden_states if inplace else torch.empty_like(hidden_states)
    if T == 0:
        return out
    tw = topk_weights.to(torch.float32).contiguous()
    ti = topk_ids.to(torch.int32).contiguous()
    dev = hidden_states.device
    nbytes = lib.moe_b200_fused_experts_workspace_bytes(T, E, k, H, inter)
    ws = _workspaces.get(dev, nbytes)
    with torch.cuda.device(dev):
        check(lib.moe_b200_fused_experts(
            hidden_states.data_ptr(), w1.data_ptr(), w2.data_ptr(),
            w1_bias.data_ptr() if w1_bias is not None else 0, w2_bias.data_ptr() if w2_bias is not None else 0,
            tw.data_ptr(), ti.data_ptr(), out.data_ptr(), T, E, k, H, inter, ACT_CODES[activation],
            ws.data_ptr(), ws.numel(), ops.status_word(dev).data_ptr(), torch.cuda.current_stream().cuda_stream))
    return out


def fused_moe_forward_reduce_norm(hidden_states: torch.Tensor, router_logits: torch.Tensor, w13: torch.Tensor,
                                  w2: torch.Tensor, top_k: int, residual: torch.Tensor, norm_weight: torch.Tensor,
                                  eps: float, comm, renormalize: bool = True, activation: str = "silu",
                                  w13_bias: Optional[torch.Tensor] = None, w2_bias: Optional[torch.Tensor] = None):
    """Router + experts + tensor-parallel reduction + the NEXT decoder layer's input_layernorm(hidden, residual)
    (nanovllm/models/qwen3_moe.py:99-116 followed by :262-270) through one library call; the k-slot sum, the
    all-reduce and the add + norm are one kernel for decode-sized batches. residual is updated in place.
    Returns (normed hidden states, residual)."""
    T, H = hidden_states.shape
    E, two_i, _ = w13.shape
    inter = two_i // 2
    assert comm is not None and not comm.disabled and comm.world_size > 1, "needs an initialised CustomAllreduce"
    assert router_logits.shape == (T, E)
    _check_experts_args(hidden_states, w13, w2, router_logits, router_logits, activation)
    assert residual.shape == (T, H) and residual.dtype == torch.bfloat16 and residual.is_contiguous()
    logits = router_logits if router_logits.dtype in (torch.bfloat16, torch.float32) else router_logits.float()
    logits = logits.contiguous()
    normed = torch.empty_like(hidden_states)
    if T == 0:
        return normed, residual
    scratch = torch.empty_like(hidden_states)
    dev = hidden_states.device
    ws = _workspaces.get(dev, lib.moe_b200_fused_moe_workspace_bytes(T, E, top_k, H, inter))
    with torch.cuda.device(dev):
        check(lib.moe_b200_fused_moe_forward_tp_add_rms_norm(
            hidden_states.data_ptr(), logits.data_ptr(), int(logits.dtype == torch.bfloat16), w13.data_ptr(),
            w2.data_ptr(), w13_bias.data_ptr() if w13_bias is not None else 0,
            w2_bias.data_ptr() if w2_bias is not None else 0, residual.data_ptr(), norm_weight.data_ptr(), float(eps),
            normed.data_ptr(), scratch.data_ptr(), T, E, top_k, H, inter, int(bool(renormalize)), ACT_CODES[activation],
            ws.data_ptr(), ws.numel(), comm._ptr, comm.buffer_ptrs[comm.rank], comm.max_size, 0,
            ops.status_word(dev).data_ptr(), torch.cuda.current_stream().cuda_stream))
    return normed, residual


def _fused_experts_fp8(hidden_states, w1, w2, topk_weights, topk_ids, inplace, activation, w1_scale, w2_scale,
                       block_shape, w1_bias, w2_bias, a1_scale, a2_scale, w1_zp, w2_zp, expert_map,
                       apply_router_weight_on_input, out: Optional[torch.Tensor] = None,
                       intermediate_offset: int = 0, intermediate_size: Optional[int] = None, comm=None) -> torch.Tensor:
    """w8a8 e4m3: weights [E, 2I, H] / [E, H, I] with fp32 scales per 128 x 128 block, activations quantised per
    token and 128 columns inside the library (dynamic, so a1_scale / a2_scale stay None)."""
    if not hidden_states.is_cuda:
        raise RuntimeError("fused_experts needs CUDA tensors; there is no CPU path")
    if hidden_states.dtype != torch.bfloat16:
        raise ValueError(f"Unsupported compute_type: {hidden_states.dtype} (activations enter as bfloat16)")
    if w2.dtype != w1.dtype:
        raise ValueError("w1 and w2 must both be e4m3")
    if w1_scale is None or w2_scale is None or block_shape is None or list(block_shape) != [128, 128]:
        raise ValueError("fp8 weights need w1_scale, w2_scale and block_shape=[128, 128]")
    if activation != "silu" or w1_bias is not None or w2_bias is not None:
        raise NotImplementedError("the fp8 path is built for silu without expert biases")
    for name, v in dict(a1_scale=a1_scale, a2_scale=a2_scale, w1_zp=w1_zp, w2_zp=w2_zp, expert_map=expert_map).items():
        assert v is None, f"{name} is not supported"
    if apply_router_weight_on_input:
        raise NotImplementedError("apply_router_weight_on_input=True is not used by the reference's models")
    assert hidden_states.is_contiguous() and w1.is_contiguous() and w2.is_contiguous()
    T, H = hidden_states.shape
    E, two_i, _ = w1.shape
    inter = two_i // 2
    assert w1.shape == (E, 2 * inter, H) and w2.shape == (E, H, inter)
    i_total = inter if intermediate_size is None else int(intermediate_size)
    i_off = int(intermediate_offset)
    if H % 128 or i_total % 128 or inter % 64 or i_off % 64 or i_off < 0 or i_off + inter > i_total:
        raise ValueError(f"fp8 path needs H and I to be multiples of 128 and a rank's slice of I to start and end "
                         f"on multiples of 64 (H={H}, I={i_total}, slice [{i_off}, {i_off + inter}))")
    s1 = w1_scale.to(torch.float32).contiguous()
    s2 = w2_scale.to(torch.float32).contiguous()
    assert s1.shape == (E, 2 * i_total // 128, H // 128), f"w1_scale shape {tuple(s1.shape)}"
    assert s2.shape == (E, H // 128, i_total // 128), f"w2_scale shape {tuple(s2.shape)}"
    k = topk_ids.size(1)
    if out is None:
        out = hidden_states if inplace else torch.empty_like(hidden_states)
    assert out.shape == hidden_states.shape and out.dtype == torch.bfloat16 and out.is_contiguous()
    if T == 0:
        return out
    tw = topk_weights.to(torch.float32).contiguous()
    ti = topk_ids.to(torch.int32).contiguous()
    dev = hidden_states.device
    nbytes = lib.moe_b200_fused_experts_fp8_workspace_bytes(T, E, k, H, inter)
    ws = _workspaces.get(dev, nbytes)
    import ctypes
    fptr = ctypes.POINTER(ctypes.c_float)
    with torch.cuda.device(dev):
        if comm is not None and not comm.disabled and comm.world_size > 1 and T * H * 2 <= comm.max_size:
            check(lib.moe_b200_fused_experts_fp8_tp_reduce(
                hidden_states.data_ptr(), w1.data_ptr(), ctypes.cast(s1.data_ptr(), fptr), w2.data_ptr(),
                ctypes.cast(s2.data_ptr(), fptr), tw.data_ptr(), ti.data_ptr(), out.data_ptr(), T, E, k, H, inter, i_off,
                i_total, ws.data_ptr(), ws.numel(), comm._ptr, comm.buffer_ptrs[comm.rank], comm.max_size, 0,
                ops.status_word(dev).data_ptr(), torch.cuda.current_stream().cuda_stream))
        else:
            check(lib.moe_b200_fused_experts_fp8_tp(
                hidden_states.data_ptr(), w1.data_ptr(), ctypes.cast(s1.data_ptr(), fptr), w2.data_ptr(),
                ctypes.cast(s2.data_ptr(), fptr), tw.data_ptr(), ti.data_ptr(), out.data_ptr(), T, E, k, H, inter, i_off,
                i_total, ws.data_ptr(), ws.numel(), ops.status_word(dev).data_ptr(),
                torch.cuda.current_stream().cuda_stream))
    return out


def shard_fp8_expert_weights(w13_q: torch.Tensor, w2_q: torch.Tensor, tp_rank: int, tp_size: int):
    """Slices e4m3 expert weights over the intermediate dimension the way FusedMoE.weight_loader slices bf16 ones
    (nanovllm/layers/fused_moe.py:400-470): w13 [E, 2I, H] -> its gate rows then its up rows of this rank, w2 [E, H, I] ->
    its columns. Returns (w13_local, w2_local, intermediate_offset); the scales are NOT sliced (the kernels index the
    unsharded scale tensors by global position). Works on any device."""
    E, two_i, _ = w13_q.shape
    inter = two_i // 2
    if inter % tp_size:
        raise ValueError(f"intermediate size {inter} is not divisible by the tensor-parallel size {tp_size}")
    ip = inter // tp_size
    lo, hi = tp_rank * ip, (tp_rank + 1) * ip
    b13, b2 = w13_q.view(torch.uint8), w2_q.view(torch.uint8)
    w13_local = torch.cat([b13[:, lo:hi], b13[:, inter + lo:inter + hi]], dim=1).contiguous().view(w13_q.dtype)
    w2_local = b2[:, :, lo:hi].contiguous().view(w2_q.dtype)
    return w13_local, w2_local, lo


def fused_experts_fp8_shard(hidden_states: torch.Tensor, w13_q: torch.Tensor, w13_scale: torch.Tensor,
                            w2_q: torch.Tensor, w2_scale: torch.Tensor, topk_weights: torch.Tensor,
                            topk_ids: torch.Tensor, intermediate_offset: int, intermediate_size: int,
                            out: Optional[torch.Tensor] = None, comm=None) -> torch.Tensor:
    """One tensor-parallel rank of the fp8 experts: w13_q [E, 2*Ip, H] / w2_q [E, H, Ip] hold the slice
    [intermediate_offset, intermediate_offset + Ip) of the intermediate dimension (sharded as FusedMoE.weight_loader
    shards bf16 weights), the scales are those of the unsharded weights. Returns this rank's partial sum, or, with
    `comm` (an initialised CustomAllreduce), the layer's output: the k-slot sum then runs inside the all-reduce."""
    return _fused_experts_fp8(hidden_states, w13_q, w2_q, topk_weights, topk_ids, False, "silu", w13_scale, w2_scale,
                              [128, 128], None, None, None, None, None, None, None, False, out=out,
                              intermediate_offset=intermediate_offset, intermediate_size=intermediate_size, comm=comm)


def pre_moe(hidden_states: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor, eps: float,
            gate_weight: torch.Tensor, top_k: int, renormalize: bool = True, return_logits: bool = False):
    """The decoder layer's steps in front of the MoE block (nanovllm/models/qwen3_moe.py:276-282 and :100-110):
    post_attention_layernorm(hidden_states, residual) -> gate -> softmax/top-k, one library call.

    hidden_states: bf16 [T, H] attention output (not modified); residual: bf16 [T, H], updated in place;
    norm_weight: RMSNorm.weight [H]; gate_weight: ReplicatedLinear.weight [E, H].
    Returns (normed hidden states, residual, topk_weights fp32 [T, k], topk_ids int32 [T, k][, router_logits bf16 [T, E]])."""
    if not hidden_states.is_cuda:
        raise RuntimeError("pre_moe needs CUDA tensors; there is no CPU path")
    for t in (hidden_states, residual, norm_weight, gate_weight):
        assert t.dtype == torch.bfloat16 and t.is_contiguous()
    T, H = hidden_states.shape
    E = gate_weight.size(0)
    assert residual.shape == (T, H) and norm_weight.numel() == H and gate_weight.shape == (E, H)
    dev = hidden_states.device
    normed = torch.empty_like(hidden_states)
    tw = torch.empty(T, top_k, dtype=torch.float32, device=dev)
    ti = torch.empty(T, top_k, dtype=torch.int32, device=dev)
    logits = torch.empty(T, E, dtype=torch.bfloat16, device=dev) if return_logits else None
    if T > 0:
        nbytes = lib.moe_b200_pre_moe_workspace_bytes(T, H, E)
        ws = _workspaces.get(dev, nbytes)
        with torch.cuda.device(dev):
            check(lib.moe_b200_add_rms_norm_router(
                hidden_states.data_ptr(), residual.data_ptr(), norm_weight.data_ptr(), float(eps), gate_weight.data_ptr(),
                normed.data_ptr(), logits.data_ptr() if logits is not None else 0, tw.data_ptr(), ti.data_ptr(), T, H, E,
                top_k, 1 if renormalize else 0, ws.data_ptr(), ws.numel(), ops.status_word(dev).data_ptr(),
                torch.cuda.current_stream().cuda_stream))
    return (normed, residual, tw, ti, logits) if return_logits else (normed, residual, tw, ti)


def fused_moe_forward_fp8(hidden_states: torch.Tensor, router_logits: torch.Tensor, w13_q: torch.Tensor,
                          w13_scale: torch.Tensor, w2_q: torch.Tensor, w2_scale: torch.Tensor, top_k: int,
                          renormalize: bool = True, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Router + fp8 experts: what FusedMoE.forward does (layers/fused_moe.py:590-612) with e4m3 block-scaled weights."""
    tw, ti, _ = fused_topk(hidden_states, router_logits, top_k, renormalize)
    return _fused_experts_fp8(hidden_states, w13_q, w2_q, tw, ti, False, "silu", w13_scale, w2_scale, [128, 128], None,
                              None, None, None, None, None, None, False, out=out)


def per_token_group_quant_fp8(x: torch.Tensor, group_size: int = 128):
    """x bf16 [rows, cols] -> (e4m3 [rows, cols], fp32 scales [rows, cols / 128]); the quantisation the fp8 path
    applies to its activations."""
    if group_size != 128:
        raise ValueError("group_size must be 128")
    if not x.is_cuda:
        raise RuntimeError("per_token_group_quant_fp8 needs a CUDA tensor; there is no CPU path")
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous() and x.size(1) % 128 == 0
    q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((x.size(0), x.size(1) // 128), dtype=torch.float32, device=x.device)
    import ctypes
    with torch.cuda.device(x.device):
        check(lib.moe_b200_quant_fp8_per_token_group(
            x.data_ptr(), x.size(0), x.size(1), q.data_ptr(), ctypes.cast(s.data_ptr(), ctypes.POINTER(ctypes.c_float)),
            torch.cuda.current_stream().cuda_stream))
    return q, s


def fused_experts(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, w1_bias: Optional[torch.Tensor],
                  w2_bias: Optional[torch.Tensor], topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                  inplace: bool = False, activation: str = "silu", apply_router_weight_on_input: bool = False,
                  per_channel_quant: bool = False, global_num_experts: int = -1,
                  expert_map: Optional[torch.Tensor] = None, w1_scale=None, w2_scale=None, w1_zp=None, w2_zp=None,
                  a1_scale=None, a2_scale=None, block_shape=None, allow_deep_gemm: bool = False) -> torch.Tensor:
    """for_moe/fused_moe.py:422-460."""
    return fused_experts_impl(hidden_states, w1, w2, topk_weights, topk_ids, inplace, activation,
                              apply_router_weight_on_input, per_channel_quant, global_num_experts, expert_map,
                              w1_scale, w2_scale, w1_zp, w2_zp, a1_scale, a2_scale, block_shape, w1_bias, w2_bias)


def fused_moe_forward(hidden_states: torch.Tensor, router_logits: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor,
                      top_k: int, renormalize: bool = True, activation: str = "silu", inplace: bool = True,
                      w13_bias: Optional[torch.Tensor] = None, w2_bias: Optional[torch.Tensor] = None,
                      comm=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Router + experts (+ tensor-parallel reduction when `comm` is an initialised CustomAllreduce) through
    one library call: what FusedMoE.forward followed by maybe_all_reduce_tensor_model_parallel does
    (nanovllm/layers/fused_moe.py:746-787, nanovllm/models/qwen3_moe.py:99-116). `out` (bf16 [T, H]) is used
    as the destination when given; otherwise the result overwrites hidden_states (inplace) or a new tensor."""
    T, H = hidden_states.shape
    E, two_i, _ = w13.shape
    inter = two_i // 2
    assert router_logits.shape == (T, E), "router_logits must be [tokens, experts]"
    _check_experts_args(hidden_states, w13, w2, router_logits, router_logits, activation)
    logits = router_logits if router_logits.dtype in (torch.bfloat16, torch.float32) else router_logits.float()
    logits = logits.contiguous()
    if out is None:
        out = hidden_states if inplace else torch.empty_like(hidden_states)
    else:
        assert out.shape == hidden_states.shape and out.dtype == hidden_states.dtype and out.is_contiguous()
    if T == 0:
        return out
    dev = hidden_states.device
    nbytes = lib.moe_b200_fused_moe_workspace_bytes(T, E, top_k, H, inter)
    ws = _workspaces.get(dev, nbytes)
    stream = torch.cuda.current_stream().cuda_stream
    b13 = w13_bias.data_ptr() if w13_bias is not None else 0
    b2 = w2_bias.data_ptr() if w2_bias is not None else 0
    with torch.cuda.device(dev):
        if comm is not None and not comm.disabled and comm.world_size > 1:
            check(lib.moe_b200_fused_moe_forward_tp(
                hidden_states.data_ptr(), logits.data_ptr(), int(logits.dtype == torch.bfloat16), w13.data_ptr(),
                w2.data_ptr(), b13, b2, out.data_ptr(), T, E, top_k, H, inter, int(bool(renormalize)),
                ACT_CODES[activation], ws.data_ptr(), ws.numel(), comm._ptr, comm.buffer_ptrs[comm.rank],
                comm.max_size, 0, ops.status_word(dev).data_ptr(), stream))
        else:
            check(lib.moe_b200_fused_moe_forward(
                hidden_states.data_ptr(), logits.data_ptr(), int(logits.dtype == torch.bfloat16), w13.data_ptr(),
                w2.data_ptr(), b13, b2, out.data_ptr(), 0, 0, T, E, top_k, H, inter, int(bool(renormalize)),
                ACT_CODES[activation], ws.data_ptr(), ws.numel(), ops.status_word(dev).data_ptr(), stream))
    return out
