"""The allocation-free decode entry point, called through its exported C symbol.

Some users of this library cannot allocate GPU memory when they need a decode step (a server that has already
given its whole memory pool away, a host language without the PyTorch allocator).  For them the library exports
``yv_paged_decode_noalloc``, which keeps its split-KV scratch in a fixed array inside the library.  This test calls
the symbol with raw pointers, twice in a row on different inputs (the second call finds the first call's leftovers
in the scratch array), and compares each result with the regular paged decode op."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from pisceslx_b200.ops import extension_path, load_extension
    load_extension()
    lib = ctypes.CDLL(str(extension_path()))
    fn = lib.yv_paged_decode_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 8 + [ctypes.c_float, ctypes.c_void_p]
    lib.yv_noalloc_strerror.restype = ctypes.c_char_p
    lib.yv_noalloc_strerror.argtypes = [ctypes.c_int]
    lib.yv_noalloc_status.restype = ctypes.c_int
    lib.yv_noalloc_status.argtypes = [ctypes.c_int, ctypes.c_void_p]
    return lib, fn


def _case(seed, lens, hq, hk, d, splits, block=64, nblocks=96, maxb=16):
    torch.manual_seed(seed)
    dev = "cuda"
    B = len(lens)
    kc = torch.randn(nblocks, block, hk, d, device=dev, dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    bt = torch.randperm(nblocks)[: B * maxb].view(B, maxb).to(torch.int32).to(dev)
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)
    q = torch.randn(B, hq, d, device=dev, dtype=torch.bfloat16)
    return q, kc, vc, bt, sl


def test_noalloc_decode_matches_regular_entry_point_twice():
    from pisceslx_b200.ops import functional as F_
    lib, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    cases = [(1, [1, 63, 64, 200, 1000], 32, 8, 128, 4), (2, [500, 7, 129], 8, 2, 64, 3)]
    for seed, lens, hq, hk, d, splits in cases:
        q, kc, vc, bt, sl = _case(seed, lens, hq, hk, d, splits)
        o = torch.zeros_like(q)
        args = (q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), sl.data_ptr(), o.data_ptr(), len(lens), hq, hk,
                d, kc.shape[1], bt.shape[1], kc.shape[0], splits, 1.0 / math.sqrt(d), stream)
        # The first launch of a kernel makes the driver load its code (lazy module loading), which moves the driver's
        # free-memory figure although nobody allocated; the figures are therefore taken around a second call.
        rc = fn(*args)
        assert rc == 0, lib.yv_noalloc_strerror(rc)
        torch.cuda.synchronize()
        o.zero_()
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]          # the driver's view: a raw cudaMalloc would move it
        rc = fn(*args)
        assert rc == 0, lib.yv_noalloc_strerror(rc)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before                  # nothing was taken from torch's allocator
        assert torch.cuda.mem_get_info()[0] >= free_before - (1 << 20)  # ... nor from the driver (scratch would be 8 MiB)
        assert lib.yv_noalloc_status(0, stream) == 0                    # no wait ran out, no index was cut
        ref = F_.paged_decode(q, kc, vc, bt, sl, splits=splits)
        # same kernels, same split count, fixed-order merge: the two entry points agree bit for bit (the regular
        # op is compared with an fp32 reference in test_gpu_kernels.py)
        assert torch.equal(o, ref), ((o.float() - ref.float()).abs().max().item())


def test_noalloc_rejects_oversized_problem():
    lib, fn = _lib()
    q, kc, vc, bt, sl = _case(3, [10, 10], 32, 8, 128, 1)
    o = torch.zeros_like(q)
    stream = torch.cuda.current_stream().cuda_stream
    # batch x heads x splits x (d + 2) far beyond the built-in capacity: rejected, nothing launched
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), sl.data_ptr(), o.data_ptr(), 4096, 32, 8, 128,
            64, bt.shape[1], kc.shape[0], 32, 0.1, stream)
    assert rc == -1 and b"capacity" in lib.yv_noalloc_strerror(rc)
    torch.cuda.synchronize()
    assert float(o.abs().sum()) == 0.0


def test_noalloc_reports_a_sequence_longer_than_its_block_table_row():
    """A length beyond max_blocks_per_seq * block is cut to the row's capacity (no read past the row) and the status
    word says so; the rows with valid lengths are unaffected."""
    from pisceslx_b200.ops import functional as F_
    lib, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    q, kc, vc, bt, sl = _case(4, [300, 1024, 40], 32, 8, 128, 2)       # row capacity: 16 blocks x 64 = 1024 tokens
    good = F_.paged_decode(q, kc, vc, bt, sl, splits=2)
    sl_bad = sl.clone()
    sl_bad[1] = 5000
    o = torch.zeros_like(q)
    assert lib.yv_noalloc_status(1, stream) == 0
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), sl_bad.data_ptr(), o.data_ptr(), 3, 32, 8, 128,
            64, bt.shape[1], kc.shape[0], 2, 1.0 / math.sqrt(128), stream)
    assert rc == 0, lib.yv_noalloc_strerror(rc)
    assert lib.yv_noalloc_status(1, stream) == 8                        # index out of range, cut
    assert lib.yv_noalloc_status(0, stream) == 0                        # cleared by the reset above
    assert torch.equal(o, good)                                         # cut to 1024 = the valid case
