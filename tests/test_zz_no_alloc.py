"""The allocation-free align entry point (``xkb_moe_align_block_size_static``), called straight
through the C ABI.  It exists for hosts that must not allocate device memory when they call in (a
plug-in inside someone else's memory pool, a serving loop with a frozen allocator): its scratch is
an array inside the library.  The outputs must equal those of the workspace-taking entry point bit
for bit, on two calls in a row (the second call finds the first call's leftovers in the shared
scratch), and sizes beyond the built-in limit must be refused with a message.

This file sorts last on purpose, so that a run stopping at the first failure has already run every
other test; it also passes when run on its own in a fresh process."""

import ctypes

import pytest
import torch

from xkernels_b200 import _lib

pytestmark = pytest.mark.gpu


def _align(lib, fn_name, ids, E, block, dev, with_workspace, expert_map=None):
    numel = ids.numel()
    max_pad = numel + (E + 1) * (block - 1)
    max_blocks = -(-max_pad // block)
    sorted_ids = torch.full((max_pad,), -7, dtype=torch.int32, device=dev)
    expert_ids = torch.full((max_blocks,), -7, dtype=torch.int32, device=dev)
    num_post = torch.full((1,), -7, dtype=torch.int32, device=dev)
    offs = torch.full((E + 1,), -7, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    emap_p = None if expert_map is None else ctypes.c_void_p(expert_map.data_ptr())
    common = [ctypes.c_void_p(ids.data_ptr()), ctypes.c_int64(numel), E, block, emap_p,
              0 if expert_map is None else expert_map.numel(),
              ctypes.c_void_p(sorted_ids.data_ptr()), ctypes.c_void_p(expert_ids.data_ptr()),
              ctypes.c_void_p(num_post.data_ptr()), ctypes.c_void_p(offs.data_ptr())]
    if with_workspace:
        nbytes = int(lib.xkb_moe_align_workspace_bytes(numel, E))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        rc = getattr(lib, fn_name)(*common, ctypes.c_void_p(ws.data_ptr()), ctypes.c_int64(nbytes), stream)
    else:
        rc = getattr(lib, fn_name)(*common, stream)
    assert rc == 0, lib.xkb_last_error()
    torch.cuda.synchronize(dev)
    return sorted_ids.cpu(), expert_ids.cpu(), num_post.cpu(), offs.cpu()


def test_static_scratch_entry_point_matches_the_workspace_one(cuda_device):
    lib = _lib.load()
    dev = cuda_device
    g = torch.Generator().manual_seed(99)
    # two calls in a row with different sizes; both use the multi-launch path (numel > 8192)
    cases = [(16384, 8, 48, 16), (5000, 4, 200, 64)]
    for M, top_k, E, block in cases:
        ids = torch.randint(0, E, (M, top_k), generator=g, dtype=torch.int32).to(dev)
        want = _align(lib, "xkb_moe_align_block_size", ids, E, block, dev, with_workspace=True)
        got = _align(lib, "xkb_moe_align_block_size_static", ids, E, block, dev, with_workspace=False)
        for a, b, name in zip(got, want, ("sorted_ids", "expert_ids", "num_post", "expert_offsets")):
            assert torch.equal(a, b), f"{name} differs for M={M} E={E}"
    # the same inputs again: identical result although the scratch still holds the previous call's data
    again = _align(lib, "xkb_moe_align_block_size_static", ids, E, block, dev, with_workspace=False)
    for a, b in zip(again, got):
        assert torch.equal(a, b)
    # the single-launch path (no scratch needed) goes through the same entry point
    small = torch.randint(0, 8, (37, 4), generator=g, dtype=torch.int32).to(dev)
    a = _align(lib, "xkb_moe_align_block_size_static", small, 8, 16, dev, with_workspace=False)
    b = _align(lib, "xkb_moe_align_block_size", small, 8, 16, dev, with_workspace=True)
    assert all(torch.equal(x, y) for x, y in zip(a, b))


def test_static_scratch_entry_point_at_its_size_limit_and_with_an_expert_map(cuda_device):
    """The largest problem the built-in array accepts (262 144 slots, 256 experts: 264 448 of its
    265 220 bytes are used) and the expert-parallel form with an expert_map, both bit for bit
    equal to the workspace entry point."""
    lib = _lib.load()
    dev = cuda_device
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 256, (32768, 8), generator=g, dtype=torch.int32).to(dev)
    want = _align(lib, "xkb_moe_align_block_size", ids, 256, 16, dev, with_workspace=True)
    got = _align(lib, "xkb_moe_align_block_size_static", ids, 256, 16, dev, with_workspace=False)
    assert all(torch.equal(a, b) for a, b in zip(got, want))
    # expert-parallel form: 64 global experts, this rank holds 16..31 as local 0..15
    emap = torch.full((64,), -1, dtype=torch.int32)
    emap[16:32] = torch.arange(16, dtype=torch.int32)
    emap = emap.to(dev)
    gids = torch.randint(0, 64, (4096, 4), generator=g, dtype=torch.int32).to(dev)
    want = _align(lib, "xkb_moe_align_block_size", gids, 16, 32, dev, with_workspace=True, expert_map=emap)
    got = _align(lib, "xkb_moe_align_block_size_static", gids, 16, 32, dev, with_workspace=False, expert_map=emap)
    assert all(torch.equal(a, b) for a, b in zip(got, want))
    assert int(got[2]) < gids.numel()      # most slots were not local and were dropped


def test_static_scratch_entry_point_refuses_oversized_problems(cuda_device):
    lib = _lib.load()
    one = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    p = ctypes.c_void_p(one.data_ptr())
    rc = lib.xkb_moe_align_block_size_static(p, ctypes.c_int64(262145), 8, 16, None, 0, p, p, p, None, None)
    assert rc == -1 and b"262144" in lib.xkb_last_error()
    rc = lib.xkb_moe_align_block_size_static(p, ctypes.c_int64(1024), 257, 16, None, 0, p, p, p, None, None)
    assert rc == -1 and b"256" in lib.xkb_last_error()
