"""Host-side mirror of the reference's row-parallel linear layer (nanovllm/layers/linear.py:155-201), the other
caller of the tensor-parallel all-reduce next to the MoE block: the attention output projection `o_proj`
(nanovllm/models/qwen3_moe.py:184-188) and the dense MLP's `down_proj`.

The product itself is a plain library GEMM (torch / cuBLAS, as in the reference). What this module adds is the
path behind it: `forward_reduce_norm` writes the GEMM result straight into the communicator's peer-visible
buffer (no staging copy) and runs the all-reduce that ends in the decoder layer's next `RMSNorm(hidden, residual)`
(nanovllm/models/qwen3_moe.py:276-282: `post_attention_layernorm` follows `o_proj`), one launch for decode-sized
batches, bit-identical to the reference's three separate steps.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from . import ops
from .custom_all_reduce import _get_ar_communicator, tensor_model_parallel_all_reduce


def divide(numerator: int, denominator: int) -> int:
    assert numerator % denominator == 0
    return numerator // denominator


class RowParallelLinear(nn.Module):
    """nanovllm/layers/linear.py:155-201: weight [output_size, input_size / tp], input sharded on its last dimension,
    partial products summed over the ranks; the bias lives on rank 0 only."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False):
        super().__init__()
        self.input_size, self.output_size, self.tp_dim = input_size, output_size, 1
        initialised = dist.is_available() and dist.is_initialized()
        self.tp_rank = dist.get_rank() if initialised else 0
        self.tp_size = dist.get_world_size() if initialised else 1
        self.input_size_per_partition = divide(input_size, self.tp_size)
        self.output_size_per_partition = output_size
        self.weight = nn.Parameter(torch.empty(self.output_size, self.input_size_per_partition), requires_grad=False)
        self.weight.weight_loader = self.weight_loader
        if bias:
            self.bias = nn.Parameter(torch.empty(self.output_size), requires_grad=False)
            self.bias.weight_loader = self.weight_loader
        else:
            self.register_parameter("bias", None)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor) -> None:
        """linear.py:176-186."""
        if param is self.bias:
            if self.tp_rank == 0:
                param.data.copy_(loaded_weight)
            return
        shard_size = param.data.size(self.tp_dim)
        param.data.copy_(loaded_weight.narrow(self.tp_dim, self.tp_rank * shard_size, shard_size))

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """linear.py:188-201."""
        if out is not None:
            if self.bias is not None and self.tp_rank == 0:
                torch.addmm(self.bias, x, self.weight.t(), out=out)
            else:
                torch.matmul(x, self.weight.t(), out=out)
            if self.tp_size > 1:
                red = tensor_model_parallel_all_reduce(out)
                if red.data_ptr() != out.data_ptr():
                    out.copy_(red)
            return out
        y = F.linear(x, self.weight, self.bias if self.tp_rank == 0 else None)
        if self.tp_size > 1:
            y = tensor_model_parallel_all_reduce(y)
        return y

    def forward_reduce_norm(self, x: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor, eps: float
                            ) -> Tuple[torch.Tensor, torch.Tensor]:
        """forward(x) followed by RMSNorm.forward(hidden, residual) of the layer that consumes it
        (nanovllm/layers/layernorm.py:21-33): returns (normed, residual), residual updated in place. With an
        initialised communicator the product is written into its peer-visible buffer and the reduction, the
        residual add and the norm are one call (one launch for decode-sized tensors)."""
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        res2 = residual.view(-1, self.output_size)
        comm = _get_ar_communicator() if self.tp_size > 1 else None
        nbytes = x2.shape[0] * self.output_size * x.element_size()
        if (comm is None or comm.disabled or x.dtype != torch.bfloat16 or nbytes > comm.max_size or x2.shape[0] == 0
                or (comm._IS_CAPTURING and not torch.cuda.is_current_stream_capturing())):
            y = self.forward(x2)
            normed = torch.empty_like(y)
            ops.add_rms_norm(normed, res2, y, norm_weight, eps)
            return normed.view(*lead, self.output_size), residual
        staged = comm.staging_view((x2.shape[0], self.output_size), torch.bfloat16)
        if self.bias is not None and self.tp_rank == 0:
            torch.addmm(self.bias, x2, self.weight.t(), out=staged)
        else:
            torch.matmul(x2, self.weight.t(), out=staged)
        normed, _ = comm.all_reduce_add_rms_norm(staged, res2, norm_weight, eps)
        return normed.view(*lead, self.output_size), residual
