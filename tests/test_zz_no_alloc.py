"""The allocation-free sort entry point (``rgs_cuda_sort_ranges_noalloc``) against the regular one.

Some users of the library cannot allocate device memory when they call into it (pre-sized real-time
loops, hosts under a fixed memory budget).  For them the sort's scratch lives inside the library image.
This test drives the entry point through its exported C symbol, twice in a row (the second call sees the
first call's leftovers in the shared scratch), and compares with ``rgs_cuda_sort_ranges``; it also checks
that a capacity beyond the built-in maximum is refused with a message.  The file name makes pytest
collect it last.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_PAIRS = 1 << 20


def _inputs(n, tiles, seed, dev):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    tile = torch.randint(0, tiles, (n,), device=dev, generator=gen, dtype=torch.int64)
    depth = torch.rand(n, device=dev, generator=gen) * 50 + 0.2
    keys = (tile << 32) | depth.view(torch.int32).to(torch.int64)
    vals = torch.randperm(n, device=dev, generator=gen).to(torch.int32)
    return keys, vals


def test_noalloc_sort_matches_regular_entry_point():
    from retinags_b200.ops import native, rasterize

    dev = torch.device("cuda")
    lib = native.lib("cuda")
    fn = lib.rgs_cuda_sort_ranges_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                   ctypes.c_void_p]
    fn.restype = ctypes.c_int
    err = lib.rgs_cuda_noalloc_last_error
    err.restype = ctypes.c_char_p
    stream = torch.cuda.current_stream(dev).cuda_stream
    for call, (n, tiles) in enumerate(((700_001, 6500), (123_457, 70_000))):
        keys, vals = _inputs(n, tiles, 11 + call, dev)
        cap = n + 77
        counters = torch.zeros(native.CNT_WORDS, dtype=torch.int32, device=dev)
        counters[native.CNT_INST] = n
        # existing entry point (caller-provided scratch)
        k0 = torch.zeros(cap, dtype=torch.int64, device=dev); k0[:n] = keys
        v0 = torch.zeros(cap, dtype=torch.int32, device=dev); v0[:n] = vals
        r0 = torch.zeros(tiles, 2, dtype=torch.int32, device=dev)
        sc = rasterize.sort_scratch(dev)
        sc.ensure(cap)
        native.call("sort_ranges", dev, k0, v0, sc.keys_tmp, sc.vals_tmp, cap, counters, tiles, r0, sc.words)
        # allocation-free entry point (scratch inside the library)
        k1 = torch.zeros(cap, dtype=torch.int64, device=dev); k1[:n] = keys
        v1 = torch.zeros(cap, dtype=torch.int32, device=dev); v1[:n] = vals
        r1 = torch.full((tiles, 2), -1, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(dev)
        reserved_before = torch.cuda.memory_reserved(dev)
        rc = fn(k1.data_ptr(), v1.data_ptr(), cap, counters.data_ptr(), tiles, r1.data_ptr(), stream)
        assert rc == 0, err().decode()
        torch.cuda.synchronize()
        if call > 0:
            # the property in the name: once the first call has resolved the scratch address (and the runtime has
            # loaded the library image), a call takes no device memory, neither from the driver nor from torch's pool
            assert torch.cuda.mem_get_info(dev)[0] == free_before
            assert torch.cuda.memory_reserved(dev) == reserved_before
        assert torch.equal(v1[:n], v0[:n])
        assert torch.equal(r1, r0)
        # and both agree with a plain stable sort
        order = torch.sort(keys, stable=True).indices
        assert torch.equal(v1[:n].long(), vals.long()[order])
    rc = fn(k1.data_ptr(), v1.data_ptr(), MAX_PAIRS + 1, counters.data_ptr(), 10, r1.data_ptr(), stream)
    assert rc == 40
    assert b"exceeds" in err()
