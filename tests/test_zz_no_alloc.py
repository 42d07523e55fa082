"""The allocation-free permutation entry point against the regular one.

Some hosts of this library cannot give `moe_b200_moe_align_block_size` the workspace it asks for: an
inference engine that has handed all remaining device memory to its KV-cache pool has nothing left to
allocate from, and a binding that mirrors the reference's op signature has no workspace argument to pass
one through. `moe_b200_moe_align_block_size_static` serves them from an array compiled into the library.
This file checks, through the C ABI, that it gives bit-identical outputs to the regular entry point on two
calls in a row (the second with different routing, so that whatever the first call left in the shared
scratch would show), that it reports requests beyond its built-in capacity instead of running, and that it
still works on small inputs. It is named so that pytest collects it after every other test file.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _routing(T, k, E, seed):
    g = torch.Generator().manual_seed(seed)
    pop = torch.rand(E, generator=g) ** 2 + 1e-3
    return torch.multinomial(pop.expand(T, E), k, replacement=False, generator=g).to(torch.int32)


def _outputs(numel, E, bs, dev):
    cap = numel + E * (bs - 1)
    return (torch.empty(cap, dtype=torch.int32, device=dev), torch.empty(-(-cap // bs), dtype=torch.int32, device=dev),
            torch.empty(1, dtype=torch.int32, device=dev))


def _regular(ids, E, bs):
    from layered_prefill_b200._lib import check, lib
    dev = ids.device
    s, e, p = _outputs(ids.numel(), E, bs, dev)
    nbytes = lib.moe_b200_align_workspace_bytes(ids.numel(), E)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    check(lib.moe_b200_moe_align_block_size(ids.data_ptr(), ids.numel(), E, bs, s.data_ptr(), s.numel(), e.data_ptr(),
                                            e.numel(), p.data_ptr(), ws.data_ptr(), nbytes,
                                            torch.cuda.current_stream().cuda_stream))
    return s, e, p


def _static(ids, E, bs):
    from layered_prefill_b200._lib import check, lib
    s, e, p = _outputs(ids.numel(), E, bs, ids.device)
    check(lib.moe_b200_moe_align_block_size_static(ids.data_ptr(), ids.numel(), E, bs, s.data_ptr(), s.numel(),
                                                   e.data_ptr(), e.numel(), p.data_ptr(),
                                                   torch.cuda.current_stream().cuda_stream))
    return s, e, p


def test_static_scratch_matches_regular_entry_point_twice_in_a_row():
    dev = torch.device("cuda", 0)
    # 8192 tokens x top-8 over 128 experts with block size 128, then a different batch and block size
    for call, (T, k, E, bs, seed) in enumerate([(8192, 8, 128, 128, 1), (5000, 8, 128, 64, 2)]):
        ids = _routing(T, k, E, seed).to(dev)
        want = _regular(ids, E, bs)
        got = _static(ids, E, bs)
        torch.cuda.synchronize()
        for name, a, b in zip(("sorted_token_ids", "expert_ids", "num_tokens_post_pad"), got, want):
            assert torch.equal(a, b), f"call {call}: {name} differs from the regular entry point"


def test_static_scratch_small_input_and_capacity_error():
    from layered_prefill_b200 import _lib
    dev = torch.device("cuda", 0)
    ids = _routing(64, 8, 128, 3).to(dev)
    want = _regular(ids, 128, 16)
    got = _static(ids, 128, 16)
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(got, want))
    # beyond the built-in capacity: a clear error, nothing launched
    assert _lib.lib.moe_b200_moe_align_static_scratch_bytes() == 33280 * 4
    big = torch.zeros(400_000, dtype=torch.int32, device=dev)
    s, e, p = _outputs(big.numel(), 256, 16, dev)
    p.fill_(-7)
    rc = _lib.lib.moe_b200_moe_align_block_size_static(big.data_ptr(), big.numel(), 256, 16, s.data_ptr(), s.numel(),
                                                       e.data_ptr(), e.numel(), p.data_ptr(),
                                                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 7 and "built-in scratch" in _lib.last_error()
    torch.cuda.synchronize()
    assert int(p.cpu()) == -7
