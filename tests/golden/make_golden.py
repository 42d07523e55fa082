"""Generates tests/golden/reference_helpers.npz from the reference's own CPU-runnable helpers.

Run where the reference tree is mounted:
    python tests/golden/make_golden.py <path of the reference tree>
It loads nanovllm/layers/for_moe/moe_easy_kernel.py by path (importing the nanovllm package itself
needs modules that are not installed) and records inputs and outputs of topk_softmax, silu_and_mul,
moe_sum and swigluoai on small seeded tensors. The tests compare the CPU oracle with these vectors;
the file is committed because the reference tree does not exist where the GPU tests run.
"""
import importlib.util
import os
import sys

import numpy as np
import torch


def load_easy_kernel(ref_root: str):
    path = os.path.join(ref_root, "nanovllm", "layers", "for_moe", "moe_easy_kernel.py")
    spec = importlib.util.spec_from_file_location("ref_moe_easy_kernel", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root: str) -> None:
    ref = load_easy_kernel(ref_root)
    g = torch.Generator().manual_seed(1234)
    out = {}

    # routing: top-k of the logits, softmax over the k picked (= renormalised softmax weights)
    for name, (T, E, k) in {"route_a": (37, 128, 8), "route_b": (5, 64, 4), "route_c": (9, 256, 8),
                            "route_d": (3, 8, 2)}.items():
        logits = torch.randn(T, E, generator=g).to(torch.bfloat16).float()
        # distinct values per row so that torch.topk's tie order does not matter
        logits = logits + torch.arange(E).float()[None, :] * 1e-3
        w = torch.empty(T, k)
        ids = torch.empty(T, k, dtype=torch.int64)
        tei = torch.empty(T, k, dtype=torch.int64)
        ref.topk_softmax(w, ids, tei, logits)
        out[f"{name}_logits"] = logits.numpy()
        out[f"{name}_weights"] = w.numpy()
        out[f"{name}_ids"] = ids.numpy().astype(np.int32)

    # gated activation, fp32 in / fp32 out (the helper's bf16 path rounds more often than the CUDA op)
    x = torch.randn(33, 2 * 64, generator=g).to(torch.bfloat16).float() * 2
    o = torch.empty(33, 64)
    ref.silu_and_mul(o, x)
    out["silu_in"] = x.numpy()
    out["silu_out"] = o.numpy()

    x = torch.randn(21, 2 * 48, generator=g).to(torch.bfloat16).float() * 4
    o = torch.empty(21, 48)
    ref.swigluoai(o, x)
    out["swiglu_in"] = x.numpy()
    out["swiglu_out"] = o.numpy()

    # k-slot sum in bf16 (fp32 accumulation inside torch.sum, one rounding)
    c3 = torch.randn(19, 8, 96, generator=g).to(torch.bfloat16)
    o = torch.empty(19, 96, dtype=torch.bfloat16)
    ref.moe_sum(c3, o)
    out["sum_in"] = c3.float().numpy()
    out["sum_out"] = o.float().numpy()

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_helpers.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT")
    if not root:
        raise SystemExit("usage: make_golden.py <path of the reference tree>   (or REFERENCE_ROOT=<path>)")
    main(root)
