"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations
(Qwen3-30B-A3B- and Qwen3-235B-A22B-shaped MoE blocks). They stand in for real checkpoints and
request traces, none of which are available offline: weights ~ N(0, 0.02), activations ~ N(0, 1),
router logits = x @ W_g^T in bf16, optionally skewed by a per-expert bias ~ N(0, 1) so that expert
load is imbalanced. Everything is drawn in fp32 from one CPU generator in a fixed order
(W_g, w13, w2, x, bias) and then cast, so a CPU checker and the GPU see identical bits.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Dict, Optional

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class MoeWorkload:
    name: str
    T: int                 # tokens in the batch
    H: int                 # hidden size
    E: int                 # experts
    top_k: int
    I: int                 # moe_intermediate_size (full, before tensor-parallel sharding)
    logit_bias_std: float = 0.0
    renormalize: bool = True
    activation: str = "silu"

    def flops(self) -> int:
        """2*T*k*3*H*I: both expert GEMMs; router GEMM and padding rows not counted."""
        return 2 * self.T * self.top_k * 3 * self.H * self.I

    def weight_bytes(self, n_active: int, tp: int = 1) -> int:
        return n_active * 3 * self.H * (self.I // tp) * 2

    def algorithmic_bytes(self, n_active: int, tp: int = 1) -> int:
        """Bytes that must cross HBM once: active experts' weights + activations in and out."""
        return self.weight_bytes(n_active, tp) + 2 * self.T * self.H * 2


WORKLOADS: Dict[str, MoeWorkload] = {
    # config 0: the reference's CPU-runnable case
    "qwen3-30b-a3b-t256": MoeWorkload("qwen3-30b-a3b-t256", 256, 2048, 128, 8, 768),
    # config 1: decode regime, weight streaming
    "qwen3-30b-a3b-decode-t64": MoeWorkload("qwen3-30b-a3b-decode-t64", 64, 2048, 128, 8, 768),
    # config 2: layered-prefill regime, imbalanced experts
    "qwen3-30b-a3b-prefill-t8192": MoeWorkload("qwen3-30b-a3b-prefill-t8192", 8192, 2048, 128, 8, 768, 1.0),
    # the chunked-prefill comparison point of config 2
    "qwen3-30b-a3b-chunk-t512": MoeWorkload("qwen3-30b-a3b-chunk-t512", 512, 2048, 128, 8, 768, 1.0),
    # config 3 shapes (run in bf16: the reference's fused_moe has no fp8 path)
    "qwen3-235b-a22b-t64": MoeWorkload("qwen3-235b-a22b-t64", 64, 4096, 128, 8, 1536),
    "qwen3-235b-a22b-t4096": MoeWorkload("qwen3-235b-a22b-t4096", 4096, 4096, 128, 8, 1536),
    # small shapes for tests
    "tiny": MoeWorkload("tiny", 17, 128, 8, 2, 64),
    "small": MoeWorkload("small", 200, 256, 16, 4, 128, 1.0),
}


def make_inputs(w: MoeWorkload, seed: int = 0, dtype: torch.dtype = torch.bfloat16,
                device: Optional[torch.device] = None) -> Dict[str, torch.Tensor]:
    """Returns W_g [E,H], w13 [E,2I,H], w2 [E,H,I], x [T,H], router_logits [T,E] (all `dtype`), and
    logit_bias [E] fp32 (zeros when the workload has no skew)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    W_g = (torch.randn(w.E, w.H, generator=g) * 0.02).to(dtype)
    w13 = torch.empty(w.E, 2 * w.I, w.H, dtype=dtype)
    for e in range(w.E):  # per expert: bounds the fp32 temporary
        w13[e] = (torch.randn(2 * w.I, w.H, generator=g) * 0.02).to(dtype)
    w2 = torch.empty(w.E, w.H, w.I, dtype=dtype)
    for e in range(w.E):
        w2[e] = (torch.randn(w.H, w.I, generator=g) * 0.02).to(dtype)
    x = torch.randn(w.T, w.H, generator=g).to(dtype)
    bias = torch.randn(w.E, generator=g) * w.logit_bias_std if w.logit_bias_std > 0 else torch.zeros(w.E)
    logits = F.linear(x, W_g)
    if w.logit_bias_std > 0:
        logits = (logits.float() + bias).to(dtype)
    out = {"W_g": W_g, "w13": w13, "w2": w2, "x": x, "router_logits": logits, "logit_bias": bias}
    if device is not None:
        out = {k: v.to(device) for k, v in out.items()}
    return out


def with_tokens(w: MoeWorkload, T: int) -> MoeWorkload:
    return replace(w, T=T, name=f"{w.name}@T{T}")
