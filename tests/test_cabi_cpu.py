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


def test_argument_errors_of_the_later_entry_points():
    """fp8 experts, the norm ops and the call in front of the block: shape and pointer checks answer before any CUDA
    call, so they can be exercised without a GPU."""
    from layered_prefill_b200 import _lib
    lib = _lib.lib
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    fp = ctypes.cast(p, ctypes.POINTER(ctypes.c_float))
    big = 1 << 34
    # fp8: H not a multiple of 128; slice of I not on a multiple of 64; slice past the end; missing workspace
    assert lib.moe_b200_fused_experts_fp8(p, p, fp, p, fp, p, p, p, 4, 8, 2, 192, 128, p, big, p, None) == 1
    assert "multiple of 128" in _lib.last_error()
    assert lib.moe_b200_fused_experts_fp8_tp(p, p, fp, p, fp, p, p, p, 4, 8, 2, 128, 192, 32, 384, p, big, p, None) == 1
    assert lib.moe_b200_fused_experts_fp8_tp(p, p, fp, p, fp, p, p, p, 4, 8, 2, 128, 192, 256, 384, p, big, p, None) == 1
    assert lib.moe_b200_fused_experts_fp8_tp(p, p, fp, p, fp, p, p, p, 4, 8, 2, 128, 192, 192, 384, p, 16, p, None) == 3
    assert "workspace" in _lib.last_error()
    assert lib.moe_b200_fused_experts_fp8_tp(p, None, fp, p, fp, p, p, p, 4, 8, 2, 128, 192, 192, 384, p, big, p, None) == 1
    assert lib.moe_b200_fused_experts_fp8_workspace_bytes(64, 128, 8, 2048, 768) > \
        lib.moe_b200_fused_experts_workspace_bytes(64, 128, 8, 2048, 768)
    assert lib.moe_b200_quant_fp8_per_token_group(p, 4, 100, p, fp, None) == 1   # row length not a multiple of 128
    # norm ops: hidden size not a multiple of 8 / above the kernel's limit; null pointers
    assert lib.moe_b200_rms_norm(p, p, p, 1e-6, 4, 100, None) == 1
    assert lib.moe_b200_add_rms_norm(p, p, p, p, 1e-6, 4, 32000, None) == 1
    assert lib.moe_b200_add_rms_norm(p, None, p, p, 1e-6, 4, 128, None) == 1
    # the call in front of the block: k > E, H not a multiple of 16, the unfused path without its workspace
    assert lib.moe_b200_add_rms_norm_router(p, p, p, 1e-6, p, p, None, fp, p, 4, 128, 8, 9, 1, p, big, p, None) == 1
    assert lib.moe_b200_add_rms_norm_router(p, p, p, 1e-6, p, p, None, fp, p, 4, 120, 8, 2, 1, p, big, p, None) == 1
    assert lib.moe_b200_add_rms_norm_router(p, p, p, 1e-6, p, p, None, fp, p, 4, 128, 16, 2, 1, None, 0, p, None) == 3
    assert lib.moe_b200_pre_moe_workspace_bytes(4096, 2048, 128) >= 4096 * 128 * 2
    # all-reduce additions: a null communicator is an argument error
    assert lib.moe_b200_ar_register_fused_buffer(0, None, 64) == 1
    assert lib.moe_b200_ar_all_reduce_add_rms_norm(0, p, p, p, p, 1e-6, p, 4, 128, p, 4096, 0, p, None) == 1
