"""The allocation-free expert sort, called through its exported C symbol.

Some callers of this library cannot allocate device memory at the point where they need the sort
(inside a CUDA-graph capture region, under a fixed memory allowance owned by another framework, in
an allocator callback). For them the library exports `cem_expert_sort_noalloc`, which runs the same
sort on a scratch array built into the library. This test loads the shared object with ctypes,
calls the symbol twice in a row on different inputs (the second call sees the first call's
leftovers in the shared scratch) and checks every output against the library's regular sort.
The file is named so that pytest collects it last.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular_sort(ext_rank, ids, num_experts):
    n = ids.numel()
    order = torch.empty(n, dtype=torch.int32, device="cuda")
    inv = torch.empty_like(order)
    counts = torch.zeros(num_experts, dtype=torch.int32, device="cuda")
    ext_rank.sort_only(ids, order, inv, counts)
    torch.cuda.synchronize()
    return order, inv, counts


def test_noalloc_expert_sort_matches_the_regular_entry_point():
    from chunked_ep_moe_b200 import ChunkedMoEConfig, _build
    from chunked_ep_moe_b200.parallel.lockstep import LockstepWorld

    _build.load()
    lib = ctypes.CDLL(_build._so_path())
    fn = lib.cem_expert_sort_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p]

    torch.cuda.set_device(0)
    num_experts, top_k, tokens = 64, 4, 3000
    cfg = ChunkedMoEConfig(num_experts=num_experts, top_k=top_k, slice_size=256, transport="nvshmem",
                           expert_compute="fused", stripe_width=64)
    world = LockstepWorld(cfg, 1, 256, 256, tokens)  # only used for its regular sort entry point
    gen = torch.Generator().manual_seed(7)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):  # two calls in a row share the built-in scratch
        n = tokens * top_k if call == 0 else 4100  # second call: different size, different block count
        ids = torch.randint(0, num_experts, (n,), generator=gen, dtype=torch.int32).cuda()
        order = torch.full((n,), -1, dtype=torch.int32, device="cuda")
        inv = torch.full((n,), -1, dtype=torch.int32, device="cuda")
        counts = torch.full((num_experts,), -1, dtype=torch.int32, device="cuda")
        rc = fn(ids.data_ptr(), n, num_experts, order.data_ptr(), inv.data_ptr(), counts.data_ptr(), stream)
        assert rc == 0, f"cem_expert_sort_noalloc returned {rc}"
        torch.cuda.synchronize()
        want_order, want_inv, want_counts = _regular_sort(world.ranks[0], ids, num_experts)
        assert torch.equal(order, want_order)
        assert torch.equal(inv, want_inv)
        assert torch.equal(counts, want_counts)
    world.close()
    # The corners of the built-in scratch: the largest problem the entry point accepts (524288 ids, 1024 experts:
    # the only case that touches the array's last entries) and the smallest (one id).
    big_cfg = ChunkedMoEConfig(num_experts=1024, top_k=8, slice_size=256, transport="nvshmem",
                               expert_compute="fused", stripe_width=64)
    world = LockstepWorld(big_cfg, 1, 256, 256, 524288 // 8)
    for n in (524288, 1):
        ids = torch.randint(0, 1024, (n,), generator=gen, dtype=torch.int32).cuda()
        order = torch.full((n,), -1, dtype=torch.int32, device="cuda")
        inv = torch.full((n,), -1, dtype=torch.int32, device="cuda")
        counts = torch.full((1024,), -1, dtype=torch.int32, device="cuda")
        assert fn(ids.data_ptr(), n, 1024, order.data_ptr(), inv.data_ptr(), counts.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        want_order, want_inv, want_counts = _regular_sort(world.ranks[0], ids, 1024)
        assert torch.equal(order, want_order) and torch.equal(inv, want_inv) and torch.equal(counts, want_counts)
    # sizes beyond the built-in scratch are refused, not truncated
    ids = torch.zeros(8, dtype=torch.int32, device="cuda")
    out = torch.zeros(8, dtype=torch.int32, device="cuda")
    assert fn(ids.data_ptr(), 524289, 8, out.data_ptr(), out.data_ptr(), out.data_ptr(), stream) == -2
    assert fn(ids.data_ptr(), 8, 1025, out.data_ptr(), out.data_ptr(), out.data_ptr(), stream) == -3
    assert fn(None, 8, 8, out.data_ptr(), out.data_ptr(), out.data_ptr(), stream) == -1
    world.close()
