"""The allocation-free compress entry point against the regular one.

b200c_btc_compress_noalloc serves hosts that cannot let the library allocate GPU memory (the whole
device is owned by the host's pool, or an allocation's device-wide synchronisation is unaffordable
while other streams run).  Its working arrays sit in a fixed buffer inside the library, shared by
all calls and never cleared between them, so the check is made on two calls in a row: a large
compressible input first, then a smaller and different one whose result would be wrong if anything
left over from the first call were read.  Both must equal what b200c_btc_compress returns, byte for
byte (integer data: no tolerance).  This file sorts last so that a run stopping at the first failure
has already been through every other test.
"""
import ctypes as C

import numpy as np
import pytest

from npu_plugin_b200 import _cabi as A
from npu_plugin_b200.const import raise_for

pytestmark = pytest.mark.gpu


class Dev:
    """Device buffer owned by the test (the entry point under test allocates nothing itself)."""

    def __init__(self, gpu, nbytes):
        self.gpu = gpu
        p = C.c_void_p()
        raise_for(gpu.lib.b200c_dev_alloc(gpu.ctx, max(1, nbytes), C.byref(p)), gpu.lib.b200c_last_error())
        self.ptr, self.n = p.value, nbytes

    def upload(self, a):
        raise_for(self.gpu.lib.b200c_memcpy_h2d(self.gpu.ctx, self.ptr, a.ctypes.data, a.size), self.gpu.lib.b200c_last_error())

    def download(self, n):
        out = np.zeros(n, np.uint8)
        raise_for(self.gpu.lib.b200c_memcpy_d2h(self.gpu.ctx, out.ctypes.data, self.ptr, n), self.gpu.lib.b200c_last_error())
        return out

    def free(self):
        self.gpu.lib.b200c_dev_free(self.gpu.ctx, self.ptr)


def compress_noalloc(gpu, x, stream=None, shift_in=0, shift_out=0):
    """The caller owns every buffer; shift_in / shift_out move the device pointers off their alignment."""
    cap = gpu.btc_bound(x.size)
    src, dst = Dev(gpu, x.size + shift_in), Dev(gpu, cap + shift_out)
    try:
        staged = np.zeros(x.size + shift_in, np.uint8)
        staged[shift_in:] = x
        src.upload(staged)
        n = C.c_size_t()
        rc = gpu.lib.b200c_btc_compress_noalloc(gpu.device, src.ptr + shift_in, x.size, dst.ptr + shift_out, cap, stream,
                                                C.byref(n))
        raise_for(rc, gpu.lib.b200c_last_error())
        return dst.download(n.value + shift_out)[shift_out:], rc == A.NOT_SMALLER
    finally:
        src.free()
        dst.free()


def test_noalloc_matches_regular_entry_point_twice_in_a_row(gpu):
    rng = np.random.default_rng(2024)
    # call 1: 3 MiB + 37 bytes of small signed values with zeros (every block mode occurs)
    a = np.clip(np.rint(rng.laplace(0, 6, 3 * (1 << 20) + 37)), -127, 127).astype(np.int8).view(np.uint8)
    a[rng.random(a.size) < 0.3] = 0
    a[4096:8192] = 7
    # call 2: shorter, incompressible noise
    b = rng.integers(0, 256, 70_001, dtype=np.uint8)
    for x in (a, b):
        ref, ref_ns = gpu.btc_compress(x)
        got, got_ns = compress_noalloc(gpu, x)
        assert got_ns == ref_ns
        assert got.size == ref.size and np.array_equal(got, ref)
        assert np.array_equal(gpu.btc_decompress(got, x.size), x)


def test_noalloc_rejects_oversized_input(gpu):
    n = A.NOALLOC_MAX_INPUT + 1
    src, dst = Dev(gpu, 16), Dev(gpu, 16)
    try:
        out_n = C.c_size_t()
        rc = gpu.lib.b200c_btc_compress_noalloc(gpu.device, src.ptr, n, dst.ptr, gpu.btc_bound(n), None, C.byref(out_n))
        assert rc == A.ERR_CAPACITY
        assert b"at most" in gpu.lib.b200c_last_error()
    finally:
        src.free()
        dst.free()


def test_noalloc_at_the_size_limit_on_a_caller_stream_with_unaligned_buffers(gpu):
    """The largest input the entry point takes (all 64 tiles of its fixed tables in use), then one a few bytes
    shorter whose device pointers are off their 16-byte alignment, both on a stream the caller created."""
    import torch
    rng = np.random.default_rng(77)
    stream = torch.cuda.Stream()
    full = np.clip(np.rint(rng.laplace(0, 9, A.NOALLOC_MAX_INPUT)), -127, 127).astype(np.int8).view(np.uint8)
    full[rng.random(full.size) < 0.2] = 0
    for x, si, so in ((full, 0, 0), (full[:full.size - 5], 1, 1), (full[:1_000_000], 3, 7)):
        ref, ref_ns = gpu.btc_compress(x)
        got, got_ns = compress_noalloc(gpu, x, stream=C.c_void_p(stream.cuda_stream), shift_in=si, shift_out=so)
        assert got_ns == ref_ns
        assert got.size == ref.size and np.array_equal(got, ref)
        assert np.array_equal(gpu.btc_decompress(got, x.size), x)


def test_noalloc_allocates_no_device_memory_and_keeps_the_current_device(gpu):
    """Free device memory is the same before and after a call once the first call has run, and the calling
    thread's current device is left as it was."""
    import torch
    x = np.arange(200_000, dtype=np.uint32).view(np.uint8)[:700_001].copy()
    cap = gpu.btc_bound(x.size)
    src, dst = Dev(gpu, x.size), Dev(gpu, cap)
    try:
        src.upload(x)
        n = C.c_size_t()
        call = lambda: gpu.lib.b200c_btc_compress_noalloc(gpu.device, src.ptr, x.size, dst.ptr, cap, None, C.byref(n))
        assert call() in (A.OK, A.NOT_SMALLER)  # first call on this device: resolves the buffer's address
        torch.cuda.synchronize()
        before_dev = torch.cuda.current_device()
        free0, _ = torch.cuda.mem_get_info(gpu.device)
        for _ in range(3):
            assert call() in (A.OK, A.NOT_SMALLER)
        free1, _ = torch.cuda.mem_get_info(gpu.device)
        assert free1 == free0, "the call changed the amount of free device memory"
        assert torch.cuda.current_device() == before_dev
    finally:
        src.free()
        dst.free()
