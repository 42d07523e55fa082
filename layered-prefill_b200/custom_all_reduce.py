"""Host-side mirror of nanovllm/layers/custom_all_reduce.py: `CustomAllreduce`,
`tensor_model_parallel_all_reduce`, `capture`, with the reference's names and call shapes, on top of
the peer-memory all-reduce of libmoe_b200.

Differences that matter to a caller:
  * the default size limit is 64 MiB instead of 8 MiB (custom_all_reduce.py:97), so the 32 MiB
    reduction of an 8192-token layered-prefill batch stays on the peer-memory kernel instead of
    falling back to NCCL (custom_all_reduce.py:253,364);
  * every device-side wait is bounded; after a wait ran out `ops.read_status()` is non-zero and the
    communicator must be closed (the reference spins forever on a lost peer);
  * `fused_moe.fused_moe_forward(..., comm=...)` runs the k-slot sum and this reduction as one launch.
"""
from __future__ import annotations

import os
from contextlib import AbstractContextManager, contextmanager
from typing import List, Optional

import torch
import torch.distributed as dist

from . import ops
from ._lib import check, lib

MiB = 1024 * 1024
DEFAULT_MAX_SIZE = 64 * MiB
FUSED_BUFFER_BYTES = 1 * MiB  # two halves of 512 KiB = the largest one-shot message at 4 ranks
LL_MAX_MESSAGE_BYTES = 256 * 1024  # decode batches: 64 tokens x 2048 hidden bf16; the receive area is 4 x world x this


def is_weak_contiguous(inp: torch.Tensor) -> bool:
    """custom_all_reduce.py:56-59."""
    return inp.is_contiguous() or (inp.untyped_storage().nbytes() - inp.storage_offset() * inp.element_size()
                                   == inp.numel() * inp.element_size())


def is_fully_connected(physical_device_ids: List[int]) -> bool:
    """NVLink (one hop) between every pair of the given GPUs, asked of NVML (custom_all_reduce.py:62-88)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        handles = [pynvml.nvmlDeviceGetHandleByIndex(i) for i in physical_device_ids]
        for i, h in enumerate(handles):
            for j, peer in enumerate(handles):
                if i < j:
                    st = pynvml.nvmlDeviceGetP2PStatus(h, peer, pynvml.NVML_P2P_CAPS_INDEX_NVLINK)
                    if st != pynvml.NVML_P2P_STATUS_OK:
                        return False
        return True
    except Exception:  # noqa: BLE001  (no NVML, or the query is not supported)
        print("NVLink detection failed. This is normal if your machine has no NVLink equipped.")
        return False


class CustomAllreduce:
    """Owner of the IPC-shared buffers and of the C-side communicator (custom_all_reduce.py:91-332)."""

    _SUPPORTED_WORLD_SIZES = [2, 4, 6, 8]

    def __init__(self, max_size: int = DEFAULT_MAX_SIZE, symm_mem_enabled: bool = False,
                 group: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None) -> None:
        self._IS_CAPTURING = False
        self.disabled = True
        self._ptr = 0
        self.gloo_group = group if group is not None else dist.new_group(backend="gloo")
        assert dist.get_backend(self.gloo_group) != dist.Backend.NCCL, \
            "CustomAllreduce should be attached to a non-NCCL group."
        rank = dist.get_rank(self.gloo_group)
        world_size = dist.get_world_size(self.gloo_group)
        self.rank = rank
        self.world_size = world_size
        if world_size == 1:
            return
        if world_size not in CustomAllreduce._SUPPORTED_WORLD_SIZES:
            print(f"Custom allreduce is disabled due to an unsupported world size: {world_size}. Supported world "
                  f"sizes: {CustomAllreduce._SUPPORTED_WORLD_SIZES}.")
            return
        if not torch.cuda.is_available():
            print("Custom allreduce is disabled because no CUDA device is present")
            return
        if device is None:
            device = torch.device(f"cuda:{int(os.environ.get('LOCAL_RANK', rank))}")
        self.device = device

        device_ids = list(range(torch.cuda.device_count()))
        if os.environ.get("CUDA_VISIBLE_DEVICES"):
            device_ids = [int(x) for x in os.environ["CUDA_VISIBLE_DEVICES"].split(",")]
        physical = torch.tensor([device_ids[device.index]], dtype=torch.int, device="cpu")
        gather_list = [torch.tensor([0], dtype=torch.int, device="cpu") for _ in range(world_size)]
        dist.all_gather(gather_list, physical, group=self.gloo_group)
        fully_connected = is_fully_connected([int(t.item()) for t in gather_list])
        if world_size > 2 and not fully_connected:
            print("Custom allreduce is disabled because it's not supported on more than two PCIe-only GPUs.")
            return

        self.disabled = False
        self.max_size = max_size
        self.fully_connected = fully_connected
        with torch.cuda.device(device):
            # metadata = flag area + scratch of the two-shot algorithm; buffer = staging area for inputs
            self.meta_ptrs = self.create_shared_buffer(ops.meta_size() + max_size, group=self.gloo_group)
            self.buffer_ptrs = self.create_shared_buffer(max_size, group=self.gloo_group)
            self.rank_data = torch.empty(8 * MiB, dtype=torch.uint8, device=device)
            self._ptr = ops.init_custom_ar(self.meta_ptrs, self.rank_data, rank, fully_connected)
            ops.register_buffer(self._ptr, self.buffer_ptrs)
            # two 512 KiB halves for the fused k-slot-sum + one-shot all-reduce (it alternates between them and
            # so needs no closing barrier); nothing else may write this buffer
            self.fused_ptrs = self.create_shared_buffer(FUSED_BUFFER_BYTES, group=self.gloo_group)
            ops.register_fused_buffer(self._ptr, self.fused_ptrs, FUSED_BUFFER_BYTES)
            # receive areas of the flag-in-data reduction: 2 parities x world source slots x 2 x message bytes
            self.ll_bytes = 4 * world_size * LL_MAX_MESSAGE_BYTES
            self.ll_ptrs = self.create_shared_buffer(self.ll_bytes, group=self.gloo_group)
            ops.register_ll_buffer(self._ptr, self.ll_ptrs, self.ll_bytes)

    @contextmanager
    def capture(self):
        """Records the addresses all-reduced inside a CUDA-graph capture and registers them with the peers
        when the context ends (custom_all_reduce.py:206-219)."""
        try:
            self._IS_CAPTURING = True
            yield
        finally:
            self._IS_CAPTURING = False
            if not self.disabled:
                self.register_graph_buffers()

    def register_graph_buffers(self) -> None:
        handle, offset = ops.get_graph_buffer_ipc_meta(self._ptr)
        world = dist.get_world_size(self.gloo_group)
        all_data = [[None, None] for _ in range(world)]
        all_data[self.rank] = [handle, offset]
        ranks = sorted(dist.get_process_group_ranks(self.gloo_group))
        for i, r in enumerate(ranks):
            dist.broadcast_object_list(all_data[i], src=r, group=self.gloo_group, device="cpu")
        ops.register_graph_buffers(self._ptr, [d[0] for d in all_data], [d[1] for d in all_data])

    def should_custom_ar(self, inp: torch.Tensor) -> bool:
        """custom_all_reduce.py:241-254."""
        if self.disabled:
            return False
        inp_size = inp.numel() * inp.element_size()
        if inp_size % 16 != 0:
            return False
        if not is_weak_contiguous(inp):
            return False
        if inp.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            return False
        if self.world_size == 2 or self.fully_connected:
            return inp_size <= self.max_size
        return False

    def all_reduce(self, inp: torch.Tensor, *, out: Optional[torch.Tensor] = None, registered: bool = False,
                   algo: int = 0) -> torch.Tensor:
        """Out-of-place all-reduce. registered=False stages the input through the pre-registered buffer."""
        if out is None:
            out = torch.empty_like(inp)
        if registered:
            ops.all_reduce(self._ptr, inp, out, 0, 0, algo)
        else:
            ops.all_reduce(self._ptr, inp, out, self.buffer_ptrs[self.rank], self.max_size, algo)
        return out

    def all_reduce_add_rms_norm(self, inp: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                                *, algo: int = 0):
        """all_reduce(inp) followed by the next layer's RMSNorm.forward(hidden, residual) (layers/layernorm.py:21-33),
        one launch for decode-sized tensors. residual is updated in place; returns (normed, residual). Bit-identical
        to the two separate steps."""
        assert inp.dtype == torch.bfloat16 and inp.dim() == 2 and inp.is_contiguous()
        assert residual.shape == inp.shape and residual.dtype == torch.bfloat16 and residual.is_contiguous()
        T, H = inp.shape
        normed = torch.empty_like(inp)
        scratch = torch.empty_like(inp)
        if T == 0:
            return normed, residual
        with torch.cuda.device(inp.device):
            check(lib.moe_b200_ar_all_reduce_add_rms_norm(
                self._ptr, inp.data_ptr(), scratch.data_ptr(), residual.data_ptr(), weight.data_ptr(), float(eps),
                normed.data_ptr(), T, H, self.buffer_ptrs[self.rank], self.max_size, algo,
                ops.status_word(inp.device).data_ptr(), torch.cuda.current_stream().cuda_stream))
        return normed, residual

    def staging_view(self, shape, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """A tensor over the start of this rank's peer-visible staging buffer (no copy, no allocation): a producer
        that writes its result here (e.g. a GEMM with out=) feeds all_reduce / all_reduce_add_rms_norm without the
        staging copy. The buffer is shared by every staged call of this communicator: use the view at once."""
        numel = 1
        for d in shape:
            numel *= int(d)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        if self.disabled or nbytes > self.max_size:
            raise ValueError(f"staging_view: {nbytes} bytes do not fit the registered buffer")

        class _Raw:  # CUDA array interface v2 over the raw device pointer (bytes; viewed as `dtype` below)
            __cuda_array_interface__ = {"shape": (max(nbytes, 1),), "typestr": "|u1",
                                        "data": (int(self.buffer_ptrs[self.rank]), False), "version": 2}
        raw = torch.as_tensor(_Raw(), device=self.device)
        return raw[:nbytes].view(dtype).view(*shape)

    def custom_all_reduce(self, input: torch.Tensor) -> Optional[torch.Tensor]:  # noqa: A002
        """custom_all_reduce.py:276-292."""
        if self.disabled or not self.should_custom_ar(input):
            return None
        if self._IS_CAPTURING:
            if torch.cuda.is_current_stream_capturing():
                return self.all_reduce(input, registered=True)
            return torch.empty_like(input)  # warm-up run before capture: same allocation pattern
        return self.all_reduce(input, registered=False)

    def close(self) -> None:
        """Collective over the CPU group: every rank closes its mappings of the peers' buffers, all ranks meet,
        and only then each frees its own allocations (a cudaFree of memory a peer still maps is deferred by the
        driver, and an unclosed mapping leaks)."""
        if not self.disabled and self._ptr:
            ops.dispose(self._ptr)
            self._ptr = 0
            self.disabled = True
            for ptrs in (self.meta_ptrs, self.buffer_ptrs, self.fused_ptrs, self.ll_ptrs):
                for i, p in enumerate(ptrs):
                    if i != self.rank and p:
                        ops.close_mem_handle(p)
            try:
                dist.barrier(group=self.gloo_group)
            except Exception:  # noqa: BLE001  (group already destroyed, or a peer is gone: free anyway)
                pass
            self.free_shared_buffer(self.meta_ptrs, rank=self.rank)
            self.free_shared_buffer(self.buffer_ptrs, rank=self.rank)
            self.free_shared_buffer(self.fused_ptrs, rank=self.rank)
            self.free_shared_buffer(self.ll_ptrs, rank=self.rank)

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass

    @staticmethod
    def create_shared_buffer(size_in_bytes: int, uncached: Optional[bool] = False,
                             group: Optional[dist.ProcessGroup] = None) -> List[int]:
        """cudaMalloc on every rank, IPC handles exchanged over the CPU group (custom_all_reduce.py:305-322)."""
        pointer, handle = ops.allocate_shared_buffer_and_handle(size_in_bytes)
        world_size = dist.get_world_size(group)
        rank = dist.get_rank(group)
        handles = [None] * world_size
        dist.all_gather_object(handles, handle, group)
        return [pointer if i == rank else ops.open_mem_handle(h) for i, h in enumerate(handles)]

    @staticmethod
    def free_shared_buffer(pointers: List[int], rank: Optional[int] = None,
                           group: Optional[dist.ProcessGroup] = None) -> None:
        if rank is None:
            rank = dist.get_rank(group)
        ops.free_shared_buffer(pointers[rank])


_ar_comm: Optional[CustomAllreduce] = None


def _get_ar_communicator() -> CustomAllreduce:
    global _ar_comm
    if _ar_comm is None:
        _ar_comm = CustomAllreduce()
    return _ar_comm


def tensor_model_parallel_all_reduce(tensor: torch.Tensor) -> torch.Tensor:
    """custom_all_reduce.py:343-366: peer-memory all-reduce when it applies, NCCL (in place) otherwise."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        out = _get_ar_communicator().custom_all_reduce(tensor)
        if out is not None:
            return out
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM)
        return tensor
    return tensor


def capture() -> AbstractContextManager:
    """custom_all_reduce.py:368-372."""
    comm = _get_ar_communicator()
    return comm.capture() if not comm.disabled else contextmanager(lambda: (yield))()
