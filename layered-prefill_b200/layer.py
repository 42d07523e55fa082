"""Host-side mirror of nanovllm/layers/fused_moe.py: the `FusedMoE` module with the reference's
constructor arguments, parameter names and layouts (`w13_weight [E, 2*I/tp, H]`, `w2_weight
[E, H, I/tp]`, optional `w13_bias`, `w2_bias`), its `weight_loader` for unquantised checkpoints,
`select_experts`, `forward` and `maybe_all_reduce_tensor_model_parallel`.

`forward` runs router + experts as one library call; with `reduce_results=True` (or through
`forward_and_reduce`) the k-slot sum and the tensor-parallel reduction are one further fused launch.
Quantised weight formats, grouped top-k and expert parallelism are not part of the reference's
running path (its asserts reject them) and raise here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import fused_moe as _fm
from .custom_all_reduce import _get_ar_communicator, tensor_model_parallel_all_reduce


def set_weight_attrs(weight: torch.Tensor, weight_attrs: Optional[dict]) -> None:
    """nanovllm/layers/for_moe/utils.py: attach loader metadata to a parameter."""
    if weight_attrs is None:
        return
    for key, value in weight_attrs.items():
        assert not hasattr(weight, key), f"Overwriting existing tensor attribute: {key}"
        setattr(weight, key, value)


@dataclass
class FusedMoEParallelConfig:
    tp_size: int
    tp_rank: int

    @staticmethod
    def make() -> "FusedMoEParallelConfig":
        """nanovllm/layers/fused_moe.py:28-32; a process without torch.distributed is one rank."""
        if dist.is_available() and dist.is_initialized():
            return FusedMoEParallelConfig(tp_size=dist.get_world_size(), tp_rank=dist.get_rank())
        return FusedMoEParallelConfig(tp_size=1, tp_rank=0)


class FusedMoE(torch.nn.Module):
    """nanovllm/layers/fused_moe.py:218-837 (the parts on the unquantised path)."""

    def __init__(self, num_experts: int, top_k: int, hidden_size: int, intermediate_size: int,
                 params_dtype: Optional[torch.dtype] = None, reduce_results: bool = False, renormalize: bool = True,
                 use_grouped_topk: bool = False, num_expert_group: Optional[int] = None,
                 topk_group: Optional[int] = None, tp_size: Optional[int] = None, ep_size: Optional[int] = None,
                 dp_size: Optional[int] = None, prefix: str = "", custom_routing_function: Optional[Callable] = None,
                 scoring_func: str = "softmax", e_score_correction_bias: Optional[torch.Tensor] = None,
                 apply_router_weight_on_input: bool = False, activation: str = "silu",
                 num_redundant_experts: int = 0, has_bias: bool = False):
        super().__init__()
        if params_dtype is None:
            params_dtype = torch.get_default_dtype()
        self.params_dtype = params_dtype
        self.moe_parallel_config = FusedMoEParallelConfig.make()
        self.global_num_experts = num_experts + num_redundant_experts
        self.local_num_experts, self.expert_map = self.global_num_experts, None
        self.layer_name = prefix
        self.top_k = top_k
        assert intermediate_size % self.tp_size == 0
        self.hidden_size = hidden_size
        self.intermediate_size_per_partition = intermediate_size // self.tp_size
        self.reduce_results = reduce_results
        self.renormalize = renormalize
        self.use_grouped_topk = use_grouped_topk
        if use_grouped_topk:
            raise NotImplementedError("grouped top-k is not on the reference's running path")
        self.custom_routing_function = custom_routing_function
        self.scoring_func = scoring_func
        if scoring_func != "softmax":
            raise ValueError("Only softmax scoring function is supported for non-grouped topk.")
        self.e_score_correction_bias = e_score_correction_bias
        self.apply_router_weight_on_input = apply_router_weight_on_input
        self.activation = activation
        self.has_bias = has_bias

        E, ip, H = self.global_num_experts, self.intermediate_size_per_partition, hidden_size
        attrs = {"weight_loader": self.weight_loader}
        self.w13_weight = torch.nn.Parameter(torch.empty(E, 2 * ip, H, dtype=params_dtype), requires_grad=False)
        set_weight_attrs(self.w13_weight, attrs)
        self.w2_weight = torch.nn.Parameter(torch.empty(E, H, ip, dtype=params_dtype), requires_grad=False)
        set_weight_attrs(self.w2_weight, attrs)
        if has_bias:
            self.w13_bias = torch.nn.Parameter(torch.zeros(E, 2 * ip, dtype=params_dtype), requires_grad=False)
            set_weight_attrs(self.w13_bias, attrs)
            self.w2_bias = torch.nn.Parameter(torch.zeros(E, H, dtype=params_dtype), requires_grad=False)
            set_weight_attrs(self.w2_bias, attrs)

    @property
    def tp_size(self) -> int:
        return self.moe_parallel_config.tp_size

    @property
    def tp_rank(self) -> int:
        return self.moe_parallel_config.tp_rank

    # ------------------------------------------------------------------ checkpoint -> parameter
    def weight_loader(self, param: torch.nn.Parameter, loaded_weight: torch.Tensor, weight_name: str, shard_id: str,
                      expert_id: int, return_success: bool = False) -> Optional[bool]:
        """nanovllm/layers/fused_moe.py:472-658, the cases an unquantised layer meets (what utils/loader.py:37-93
        feeds it):
          * per-expert 2-D tensors, "weight" in the name: gate rows ("w1") fill the first half of w13[e], up rows
            ("w3") the second half, each narrowed to this rank's slice of I (:398-414); down ("w2") is narrowed on
            its input dimension (:416-432);
          * all-expert 3-D tensors (gpt-oss: "gate_up_proj_blocks" / "down_proj_blocks" after dequantisation), shard
            "w13": rows [rank * 2I/tp, (rank+1) * 2I/tp) of the fused, interleaved gate_up rows (:388-392); "w2":
            this rank's slice of the last dimension;
          * biases come as all-expert tensors too: "w2" is copied on rank 0 only, anything else is this rank's
            contiguous slice of the last dimension (:647-654);
          * shard "all": the whole parameter at once (:479-487)."""
        if shard_id == "all":
            if "bias" in weight_name:
                param.data.copy_(loaded_weight)
            else:
                param.data.copy_(loaded_weight.reshape(*param.data.shape[:-1], -1))
            return True if return_success else None
        if shard_id not in ("w1", "w2", "w3", "all", "w13"):
            raise ValueError(f"shard_id must be ['w1','w2','w3', 'all'] but got {shard_id}.")
        tp_rank, tp_size = self.tp_rank, self.tp_size
        full_load = loaded_weight.dim() == 3 or "bias" in weight_name or "block" in weight_name
        expert_data = param.data if full_load else param.data[expert_id]
        if "weight" in weight_name or "block" in weight_name:
            if "weight" in weight_name:
                shard_dim = {"w1": 0, "w2": 1, "w3": 0, "w13": 1}[shard_id] + (1 if full_load else 0)
            else:
                shard_dim = -1
            if expert_data.dim() != loaded_weight.dim():
                loaded_weight = loaded_weight.reshape(*loaded_weight.shape[:-2], -1)
            if shard_id == "w2":
                shard = expert_data.shape[shard_dim]
                expert_data.copy_(loaded_weight.narrow(shard_dim, shard * tp_rank, shard))
            elif shard_id in ("w1", "w3"):
                shard = expert_data.shape[shard_dim] // 2
                sl = loaded_weight.narrow(shard_dim, shard * tp_rank, shard)
                expert_data.narrow(shard_dim, 0 if shard_id == "w1" else shard, shard).copy_(sl)
            else:  # "w13": the fused gate_up rows, sharded on the output dimension
                shard = expert_data.shape[1]
                expert_data.narrow(1, 0, shard).copy_(loaded_weight.narrow(1, shard * tp_rank, shard))
            return True if return_success else None
        if "bias" in weight_name:
            if shard_id == "w2":
                if tp_rank == 0:
                    expert_data.copy_(loaded_weight)
            else:
                n = loaded_weight.size(-1)
                expert_data.copy_(loaded_weight.narrow(-1, tp_rank * n // tp_size, n // tp_size))
            return True if return_success else None
        raise ValueError(f"Unrecognized weight_name {weight_name}.")

    @classmethod
    def make_expert_params_mapping(cls, ckpt_gate_proj_name: str, ckpt_down_proj_name: str, ckpt_up_proj_name: str,
                                   num_experts: int, num_redundant_experts: int = 0):
        """nanovllm/layers/fused_moe.py:789-822: (param_name, weight_name, expert_id, shard_id) tuples."""
        n = num_experts + num_redundant_experts
        logical = list(range(num_experts)) + [i % num_experts for i in range(num_redundant_experts)]
        return [("experts.w13_" if wn in (ckpt_gate_proj_name, ckpt_up_proj_name) else "experts.w2_",
                 f"experts.{logical[e]}.{wn}.", e, sid)
                for e in range(n)
                for sid, wn in (("w1", ckpt_gate_proj_name), ("w2", ckpt_down_proj_name), ("w3", ckpt_up_proj_name))]

    # ------------------------------------------------------------------ forward
    @staticmethod
    def select_experts(hidden_states: torch.Tensor, router_logits: torch.Tensor, top_k: int, use_grouped_topk: bool,
                       renormalize: bool, topk_group: Optional[int] = None, num_expert_group: Optional[int] = None,
                       custom_routing_function: Optional[Callable] = None, scoring_func: str = "softmax",
                       e_score_correction_bias: Optional[torch.Tensor] = None,
                       indices_type: Optional[torch.dtype] = None, **_unused):
        """nanovllm/layers/fused_moe.py:693-741."""
        if custom_routing_function is None:
            topk_weights, topk_ids, _ = _fm.fused_topk(hidden_states, router_logits, top_k, renormalize)
        else:
            topk_weights, topk_ids = custom_routing_function(hidden_states=hidden_states, gating_output=router_logits,
                                                             topk=top_k, renormalize=renormalize)
            if indices_type is not None:
                topk_ids = topk_ids.to(dtype=indices_type)
        return topk_weights, topk_ids

    def maybe_all_reduce_tensor_model_parallel(self, final_hidden_states: torch.Tensor) -> torch.Tensor:
        """nanovllm/layers/fused_moe.py:746-748."""
        return tensor_model_parallel_all_reduce(final_hidden_states)

    def _bias(self, name: str) -> Optional[torch.Tensor]:
        return getattr(self, name) if self.has_bias else None

    def forward(self, hidden_states: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        """nanovllm/layers/fused_moe.py:750-787; the result overwrites hidden_states (inplace=True, :211)."""
        if self.custom_routing_function is not None:
            tw, ti = self.select_experts(hidden_states, router_logits, self.top_k, False, self.renormalize,
                                         custom_routing_function=self.custom_routing_function)
            out = _fm.fused_experts(hidden_states, self.w13_weight, self.w2_weight, self._bias("w13_bias"),
                                    self._bias("w2_bias"), tw, ti, inplace=True, activation=self.activation)
            if self.reduce_results and self.tp_size > 1:
                out = self.maybe_all_reduce_tensor_model_parallel(out)
            return out
        comm = _get_ar_communicator() if (self.reduce_results and self.tp_size > 1) else None
        if comm is not None and (comm.disabled or hidden_states.numel() * 2 > comm.max_size):
            comm = None
        out = _fm.fused_moe_forward(hidden_states, router_logits, self.w13_weight, self.w2_weight, self.top_k,
                                    self.renormalize, self.activation, inplace=True,
                                    w13_bias=self._bias("w13_bias"), w2_bias=self._bias("w2_bias"), comm=comm)
        if comm is None and self.reduce_results and self.tp_size > 1:
            out = self.maybe_all_reduce_tensor_model_parallel(out)
        return out

    def forward_and_reduce(self, hidden_states: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        """forward followed by maybe_all_reduce_tensor_model_parallel, as Qwen3MoeSparseMoeBlock.forward calls
        them back to back (nanovllm/models/qwen3_moe.py:104-114), with the sum and the reduction fused."""
        saved = self.reduce_results
        self.reduce_results = True
        try:
            return self.forward(hidden_states, router_logits)
        finally:
            self.reduce_results = saved

    def forward_reduce_norm(self, hidden_states: torch.Tensor, router_logits: torch.Tensor, residual: torch.Tensor,
                            norm_weight: torch.Tensor, eps: float):
        """forward + all-reduce + the next decoder layer's input_layernorm(hidden, residual)
        (nanovllm/models/qwen3_moe.py:262-270): returns (normed, residual) with residual updated in place. Falls back
        to the separate steps when the tensor-parallel communicator cannot take the tensor."""
        comm = _get_ar_communicator() if self.tp_size > 1 else None
        usable = (comm is not None and not comm.disabled and hidden_states.numel() * 2 <= comm.max_size
                  and self.custom_routing_function is None)
        if usable:
            return _fm.fused_moe_forward_reduce_norm(hidden_states, router_logits, self.w13_weight, self.w2_weight,
                                                     self.top_k, residual, norm_weight, eps, comm, self.renormalize,
                                                     self.activation, self._bias("w13_bias"), self._bias("w2_bias"))
        out = self.forward_and_reduce(hidden_states, router_logits) if self.tp_size > 1 else self.forward(hidden_states, router_logits)
        from . import ops as _ops
        normed = torch.empty_like(out)
        _ops.add_rms_norm(normed, residual, out, norm_weight, eps)
        return normed, residual

    def extra_repr(self) -> str:
        return (f"global_num_experts={self.global_num_experts}, top_k={self.top_k}, "
                f"intermediate_size_per_partition={self.intermediate_size_per_partition}, tp_size={self.tp_size}, "
                f"reduce_results={self.reduce_results}, renormalize={self.renormalize}, "
                f"activation='{self.activation}'")
