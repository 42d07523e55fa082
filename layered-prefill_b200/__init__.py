"""B200-native (sm_100a) implementation of the MoE-block hot path of scale-snu/layered-prefill:
router top-k softmax, moe_align_block_size, grouped gate_up/down expert GEMMs on tcgen05 with fused
activation and routed-weight combine, and the tensor-parallel all-reduce over NVLink peer memory.

Modules mirror the reference's layout for this path:
  ops               <-> nanovllm.ops (csrc/ops.cpp)            raw ops on torch tensors
  fused_moe         <-> nanovllm/layers/for_moe/fused_moe.py   fused_topk, moe_align_block_size, fused_experts
  layer             <-> nanovllm/layers/fused_moe.py           FusedMoE module
  custom_all_reduce <-> nanovllm/layers/custom_all_reduce.py   CustomAllreduce, tensor_model_parallel_all_reduce
  workload                                                      seeded synthetic inputs of the benchmark configs
Everything runs through libmoe_b200.so (C ABI in include/moe_b200.h); there is no CPU fallback.
"""
__version__ = "0.1.0"
