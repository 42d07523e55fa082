"""Host-side mirror of the hot-path functions of the reference's `nanovllm.ops` extension
(csrc/ops.cpp:97-159): same names, same argument order, torch tensors in, results written in place.
Each function forwards raw pointers to libmoe_b200 on the current CUDA stream; there is no
fallback -- a CPU tensor or a missing library is an error.
"""
from __future__ import annotations

import ctypes
from typing import List, Tuple

import torch

from . import _lib
from ._lib import check, lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("libmoe_b200 ops take CUDA tensors only (there is no CPU path)")


_status_words: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """One zero-initialised int32 per device; kernels store a code there when a bounded wait runs out."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status_words:
        _status_words[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status_words[idx]


def launch_count() -> int:
    """Kernels this library has launched in this process so far (graph replays are not seen)."""
    return int(lib.moe_b200_launch_count())


def read_status(device: torch.device | None = None) -> int:
    """Synchronise the current stream and return the device status word (0 = no device-side timeout)."""
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    v = ctypes.c_int32(0)
    with torch.cuda.device(dev):
        check(lib.moe_b200_read_status(status_word(dev).data_ptr(), ctypes.byref(v), _stream()))
    return int(v.value)


def _norm_args(out: torch.Tensor, input: torch.Tensor, weight: torch.Tensor):  # noqa: A002
    _need_cuda(out, input, weight)
    if input.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise RuntimeError("rms_norm: bfloat16 tensors only")
    assert input.is_contiguous() and out.is_contiguous() and weight.is_contiguous() and out.shape == input.shape
    H = input.size(-1)
    assert weight.numel() == H
    return (input.numel() // H if H else 0), H


def rms_norm(out: torch.Tensor, input: torch.Tensor, weight: torch.Tensor, epsilon: float) -> None:  # noqa: A002
    """csrc/ops.cpp:16-21. out = bf16(bf16(x * rsqrt(mean(x^2) + eps)) * weight); out may be input."""
    T, H = _norm_args(out, input, weight)
    with torch.cuda.device(input.device):
        check(lib.moe_b200_rms_norm(out.data_ptr(), input.data_ptr(), weight.data_ptr(), float(epsilon), T, H, _stream()))


def add_rms_norm(out: torch.Tensor, residual: torch.Tensor, input: torch.Tensor, weight: torch.Tensor,  # noqa: A002
                 epsilon: float) -> None:
    """csrc/ops.cpp:22-27. residual <- bf16(input + residual) in place, out = its RMS norm times weight."""
    T, H = _norm_args(out, input, weight)
    _need_cuda(residual)
    assert residual.dtype == torch.bfloat16 and residual.is_contiguous() and residual.shape == input.shape
    with torch.cuda.device(input.device):
        check(lib.moe_b200_add_rms_norm(out.data_ptr(), residual.data_ptr(), input.data_ptr(), weight.data_ptr(),
                                        float(epsilon), T, H, _stream()))


def topk_softmax(topk_weights: torch.Tensor, topk_indices: torch.Tensor, token_expert_indices: torch.Tensor,
                 gating_output: torch.Tensor) -> None:
    """csrc/ops.cpp:46-51. gating_output fp32 (or bf16) [T, E]; outputs [T, k]."""
    _need_cuda(topk_weights, topk_indices, token_expert_indices, gating_output)
    assert gating_output.is_contiguous() and topk_weights.is_contiguous() and topk_indices.is_contiguous()
    assert topk_weights.dtype == torch.float32 and topk_indices.dtype == torch.int32
    if gating_output.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("topk_softmax: gating_output must be float32 or bfloat16")
    E = gating_output.size(-1)
    T = gating_output.numel() // E if E else 0
    k = topk_weights.size(-1)
    tei = 0
    if token_expert_indices is not None:
        assert token_expert_indices.dtype == torch.int32 and token_expert_indices.is_contiguous()
        tei = token_expert_indices.data_ptr()
    with torch.cuda.device(gating_output.device):
        check(lib.moe_b200_topk_softmax(gating_output.data_ptr(), int(gating_output.dtype == torch.bfloat16),
                                        topk_weights.data_ptr(), topk_indices.data_ptr(), tei, T, E, k, 0, _stream()))


def topk_softmax_renorm(topk_weights: torch.Tensor, topk_indices: torch.Tensor, gating_output: torch.Tensor,
                        renormalize: bool) -> None:
    """topk_softmax with the renormalisation of fused_topk folded in (one launch, bf16 or fp32 logits)."""
    _need_cuda(topk_weights, topk_indices, gating_output)
    assert gating_output.is_contiguous() and topk_weights.is_contiguous() and topk_indices.is_contiguous()
    E = gating_output.size(-1)
    T = gating_output.numel() // E if E else 0
    with torch.cuda.device(gating_output.device):
        check(lib.moe_b200_topk_softmax(gating_output.data_ptr(), int(gating_output.dtype == torch.bfloat16),
                                        topk_weights.data_ptr(), topk_indices.data_ptr(), 0, T, E,
                                        topk_weights.size(-1), int(bool(renormalize)), _stream()))


def moe_align_block_size(topk_ids: torch.Tensor, num_experts: int, block_size: int, sorted_token_ids: torch.Tensor,
                         experts_ids: torch.Tensor, num_tokens_post_pad: torch.Tensor) -> None:
    """csrc/ops.cpp:53-60."""
    _need_cuda(topk_ids, sorted_token_ids, experts_ids, num_tokens_post_pad)
    if topk_ids.dtype != torch.int32:
        raise RuntimeError("moe_align_block_size: topk_ids must be int32")
    assert topk_ids.is_contiguous() and sorted_token_ids.is_contiguous() and experts_ids.is_contiguous()
    numel = topk_ids.numel()
    ws_bytes = lib.moe_b200_align_workspace_bytes(numel, num_experts)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=topk_ids.device)
    with torch.cuda.device(topk_ids.device):
        check(lib.moe_b200_moe_align_block_size(topk_ids.data_ptr(), numel, num_experts, block_size,
                                                sorted_token_ids.data_ptr(), sorted_token_ids.numel(),
                                                experts_ids.data_ptr(), experts_ids.numel(),
                                                num_tokens_post_pad.data_ptr(), ws.data_ptr(), ws_bytes, _stream()))


def silu_and_mul(out: torch.Tensor, input: torch.Tensor) -> None:  # noqa: A002
    """csrc/ops.cpp:29-31. input [N, 2d] -> out [N, d], bf16."""
    _need_cuda(out, input)
    if input.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise RuntimeError("silu_and_mul: bfloat16 only")
    assert input.is_contiguous() and out.is_contiguous()
    d = input.size(-1) // 2
    rows = input.numel() // (2 * d) if d else 0
    with torch.cuda.device(input.device):
        check(lib.moe_b200_silu_and_mul(out.data_ptr(), input.data_ptr(), rows, d, _stream()))


def swigluoai_and_mul(out: torch.Tensor, input: torch.Tensor, alpha: float = 1.702, limit: float = 7.0) -> None:  # noqa: A002
    """csrc/ops.cpp:33-36."""
    _need_cuda(out, input)
    if input.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise RuntimeError("swigluoai_and_mul: bfloat16 only")
    assert input.is_contiguous() and out.is_contiguous()
    d = input.size(-1) // 2
    rows = input.numel() // (2 * d) if d else 0
    with torch.cuda.device(input.device):
        check(lib.moe_b200_swigluoai_and_mul(out.data_ptr(), input.data_ptr(), rows, d, alpha, limit, _stream()))


def moe_sum(input: torch.Tensor, output: torch.Tensor) -> None:  # noqa: A002
    """nanovllm/layers/for_moe/moe_easy_kernel.py:26-31. input [T, k, H] -> output [T, H], bf16."""
    _need_cuda(input, output)
    assert input.dtype == torch.bfloat16 and output.dtype == torch.bfloat16
    assert input.is_contiguous() and output.is_contiguous()
    T, k, H = input.shape
    with torch.cuda.device(input.device):
        check(lib.moe_b200_moe_sum(input.data_ptr(), output.data_ptr(), T, k, H, _stream()))


# ---------------------------------------------------------------- custom all-reduce (csrc/ops.cpp:77-95)
def meta_size() -> int:
    return int(lib.moe_b200_ar_meta_size())


def allocate_shared_buffer_and_handle(size: int) -> Tuple[int, bytes]:
    ptr = ctypes.c_int64(0)
    handle = (ctypes.c_uint8 * 64)()
    check(lib.moe_b200_ar_allocate_shared_buffer(size, ctypes.byref(ptr), handle))
    return int(ptr.value), bytes(handle)


def open_mem_handle(handle: bytes) -> int:
    buf = (ctypes.c_uint8 * 64).from_buffer_copy(bytes(handle))
    ptr = ctypes.c_int64(0)
    check(lib.moe_b200_ar_open_mem_handle(buf, ctypes.byref(ptr)))
    return int(ptr.value)


def close_mem_handle(ptr: int) -> None:
    """Unmaps a peer's buffer opened with open_mem_handle (the reference leaves this to process exit)."""
    check(lib.moe_b200_ar_close_mem_handle(int(ptr)))


def free_shared_buffer(ptr: int) -> None:
    check(lib.moe_b200_ar_free_shared_buffer(ptr))


def init_custom_ar(ipc_ptrs: List[int], rank_data: torch.Tensor, rank: int, fully_connected: bool) -> int:
    n = len(ipc_ptrs)
    arr = (ctypes.c_int64 * n)(*ipc_ptrs)
    h = ctypes.c_int64(0)
    with torch.cuda.device(rank_data.device):
        check(lib.moe_b200_ar_init(arr, n, rank_data.data_ptr(), rank_data.numel() * rank_data.element_size(), rank,
                                   int(fully_connected), ctypes.byref(h)))
    return int(h.value)


def dispose(fa: int) -> None:
    check(lib.moe_b200_ar_dispose(fa))


def register_buffer(fa: int, ipc_ptrs: List[int]) -> None:
    arr = (ctypes.c_int64 * len(ipc_ptrs))(*ipc_ptrs)
    check(lib.moe_b200_ar_register_buffer(fa, arr))


def register_fused_buffer(fa: int, ipc_ptrs: List[int], nbytes: int) -> None:
    """A second registered buffer, used only by the fused k-slot-sum + one-shot all-reduce (two halves in alternation,
    which saves that kernel its closing barrier). No reference counterpart."""
    arr = (ctypes.c_int64 * len(ipc_ptrs))(*ipc_ptrs)
    check(lib.moe_b200_ar_register_fused_buffer(fa, arr, nbytes))


def register_ll_buffer(fa: int, ipc_ptrs: List[int], nbytes: int) -> None:
    """The receive areas of the flag-in-data one-shot reduction (data and flag travel in the same 8 bytes, no
    barrier). No reference counterpart."""
    arr = (ctypes.c_int64 * len(ipc_ptrs))(*ipc_ptrs)
    check(lib.moe_b200_ar_register_ll_buffer(fa, arr, nbytes))


_AR_DTYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def all_reduce(fa: int, inp: torch.Tensor, out: torch.Tensor, reg_buffer: int, reg_buffer_sz_bytes: int,
               algo: int = 0) -> None:
    _need_cuda(inp, out)
    if inp.dtype not in _AR_DTYPES or out.dtype != inp.dtype:
        raise RuntimeError("all_reduce: bf16/fp16/fp32 tensors of equal dtype only")
    if inp.numel() != out.numel():
        raise RuntimeError("all_reduce: input and output sizes differ")
    with torch.cuda.device(inp.device):
        check(lib.moe_b200_ar_all_reduce(fa, inp.data_ptr(), out.data_ptr(), inp.numel(), _AR_DTYPES[inp.dtype],
                                         reg_buffer, reg_buffer_sz_bytes, algo, status_word(inp.device).data_ptr(),
                                         _stream()))


def get_graph_buffer_ipc_meta(fa: int) -> Tuple[bytes, List[int]]:
    n = ctypes.c_int(0)
    check(lib.moe_b200_ar_graph_buffer_count(fa, ctypes.byref(n)))
    cnt = int(n.value)
    handles = (ctypes.c_uint8 * (64 * max(cnt, 1)))()
    offsets = (ctypes.c_int64 * max(cnt, 1))()
    check(lib.moe_b200_ar_get_graph_buffer_ipc_meta(fa, handles, offsets, cnt))
    return bytes(handles)[: 64 * cnt], [int(offsets[i]) for i in range(cnt)]


def register_graph_buffers(fa: int, handles: List[bytes], offsets: List[List[int]]) -> None:
    world = len(handles)
    cnt = len(offsets[0]) if offsets else 0
    flat_h = b"".join(bytes(h) for h in handles)
    hb = (ctypes.c_uint8 * max(len(flat_h), 1)).from_buffer_copy(flat_h if flat_h else b"\0")
    flat_o = [o for per_rank in offsets for o in per_rank]
    ob = (ctypes.c_int64 * max(len(flat_o), 1))(*flat_o) if flat_o else (ctypes.c_int64 * 1)()
    assert len(flat_h) == world * cnt * 64
    check(lib.moe_b200_ar_register_graph_buffers(fa, hb, ob, cnt))


__all__ = [
    "topk_softmax", "topk_softmax_renorm", "moe_align_block_size", "silu_and_mul", "swigluoai_and_mul", "moe_sum",
    "meta_size", "allocate_shared_buffer_and_handle", "open_mem_handle", "free_shared_buffer", "init_custom_ar",
    "dispose", "register_buffer", "all_reduce", "get_graph_buffer_ipc_meta", "register_graph_buffers",
    "status_word", "read_status",
]
_ = _lib
