"""The C-ABI library loads without a GPU and exports exactly what include/moe_b200.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "moe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(moe_b200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    from layered_prefill_b200 import _lib
    names = _declared()
    assert len(names) >= 25
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} declared in include/moe_b200.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_constants():
    from layered_prefill_b200 import _lib
    assert _lib.lib.moe_b200_abi_version() == 1
    assert _lib.lib.moe_b200_block_m() == 128
    assert _lib.lib.moe_b200_ar_meta_size() % 256 == 0


def test_workspace_sizes_are_monotone_and_cover_the_intermediates():
    from layered_prefill_b200 import _lib
    f = _lib.lib.moe_b200_fused_experts_workspace_bytes
    small, big = f(64, 128, 8, 2048, 768), f(8192, 128, 8, 2048, 768)
    assert 0 < small < big
    numel = 8192 * 8
    rows = numel + 128 * 127
    assert big >= rows * 768 * 2 + numel * 2048 * 2
    assert _lib.lib.moe_b200_fused_moe_workspace_bytes(64, 128, 8, 2048, 768) > small
    assert f(0, 0, 8, 2048, 768) == 0


def test_argument_errors_come_back_as_status_and_message():
    from layered_prefill_b200 import _lib
    lib = _lib.lib
    # all of these are rejected before any CUDA call
    assert lib.moe_b200_topk_softmax(None, 0, None, None, None, 4, 8, 2, 0, None) == 1
    assert "null" in _lib.last_error()
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    assert lib.moe_b200_topk_softmax(p, 0, p, p, None, 4, 8, 9, 0, None) == 1  # k > E
    assert lib.moe_b200_fused_experts(p, p, p, None, None, p, p, p, 4, 8, 2, 100, 64, 0, p, 1 << 30, p, None) == 1
    assert "multiples of 16" in _lib.last_error()
    assert lib.moe_b200_fused_experts(p, p, p, None, None, p, p, p, 4, 8, 2, 128, 64, 0, p, 16, p, None) == 3
    assert "workspace" in _lib.last_error()
    assert lib.moe_b200_fused_experts(p, p, p, None, None, p, p, p, 4, 8, 2, 128, 64, 5, p, 1 << 30, p, None) == 1
    assert lib.moe_b200_moe_align_block_size(p, 16, 2000, 4, p, 1 << 20, p, 1 << 20, p, None, 0, None) == 1
    assert lib.moe_b200_moe_align_block_size(p, 16, 8, 4, p, 10, p, 100, p, None, 0, None) == 1
    with pytest.raises(_lib.MoeB200Error):
        _lib.check(lib.moe_b200_ar_all_reduce(0, p, p, 8, 0, 0, 0, 0, p, None))


def test_host_mirror_rejects_cpu_tensors():
    import torch
    from layered_prefill_b200 import fused_moe, ops
    x = torch.zeros(4, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        ops.silu_and_mul(torch.zeros(4, 64, dtype=torch.bfloat16), x)
    w13 = torch.zeros(2, 64, 128, dtype=torch.bfloat16)
    w2 = torch.zeros(2, 128, 32, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        fused_moe.fused_experts(x, w13, w2, None, None, torch.zeros(4, 1), torch.zeros(4, 1, dtype=torch.int32))
    with pytest.raises(ValueError):
        fused_moe.fused_experts(x.float(), w13, w2, None, None, torch.zeros(4, 1), torch.zeros(4, 1, dtype=torch.int32))
