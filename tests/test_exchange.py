"""The exchange primitives of the multi-GPU fold on one device, and the whole sharded fold on two.

One device: the copy kernel and the copy-engine form move the same bytes (aligned and unaligned
segments) and raise the done flag; the bounded waits run out when nothing sets their flag -- the kernel
records the time-out and returns, the context stays usable, and a pusher whose release never comes
stores nothing.  Two devices (skipped on a single-GPU box): two processes fold a model through
ShardedFolder + PushTransport, and the blob assembled on rank 0 equals the single-rank blob per constant.
"""
import os
import sys
import time

import numpy as np
import pytest

from npu_plugin_b200 import _cabi as A

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_copy_segments_and_flags(gpu, mode):
    rng = np.random.default_rng(8)
    n = 3_000_000
    src_host = rng.integers(0, 256, n, dtype=np.uint8)
    src, dst, flags = gpu.dev_alloc(n), gpu.dev_alloc(n), gpu.dev_alloc(256)
    try:
        gpu.upload(src, src_host)
        gpu.fill_zero(dst, n)
        gpu.fill_zero(flags, 256)
        # (offset in src, offset in dst, bytes): aligned, unaligned source, unaligned destination, tiny, empty
        segs = [(0, 0, 1 << 20), ((1 << 20) + 1, (1 << 20) + 16, 300_001), (1_500_000, 1_500_003, 77), (2_000_000, 2_000_000, 5),
                (2_500_000, 2_500_000, 0)]
        gpu.copy_segments_async([(src + a, dst + b, k) for a, b, k in segs], done_flag=flags, done_value=7, mode=mode, ctas=16)
        gpu.wait_flags(flags, 1, 7, timeout_ms=2000)
        assert gpu.exchange_status() == 0
        got = gpu.download(dst, n)
        want = np.zeros(n, np.uint8)
        for a, b, k in segs:
            want[b:b + k] = src_host[a:a + k]
        assert np.array_equal(got, want)
        assert gpu.download(flags, 8).view(np.uint64)[0] == 7
        # a later, larger sequence value satisfies a wait for a smaller one
        gpu.wait_flags(flags, 1, 3, timeout_ms=2000)
        assert gpu.exchange_status() == 0
    finally:
        for p in (src, dst, flags):
            gpu.dev_free(p)


def test_bounded_waits_run_out_and_report(gpu):
    src, dst, flags = gpu.dev_alloc(4096), gpu.dev_alloc(4096), gpu.dev_alloc(256)
    try:
        gpu.upload(src, np.full(4096, 0x5A, np.uint8))
        gpu.fill_zero(dst, 4096)
        gpu.fill_zero(flags, 256)
        # rank 0's side: nothing ever sets flags[1..3]
        t0 = time.time()
        gpu.wait_flags(flags + 8, 3, 1, timeout_ms=300)
        assert gpu.exchange_status() & 2
        assert time.time() - t0 < 5.0
        assert gpu.exchange_status() == 0  # reading the status clears it
        # a pusher's side: the release never comes -> nothing is stored, no done flag is raised
        for mode in (0, 2):
            gpu.copy_segments_async([(src, dst, 4096)], wait_flag=flags + 64, wait_value=1, done_flag=flags, done_value=9,
                                    timeout_ms=300, mode=mode, ctas=4)
            assert gpu.exchange_status() & 1
            assert not gpu.download(dst, 4096).any()
            assert gpu.download(flags, 8).view(np.uint64)[0] == 0
        # the context is still usable
        gpu.copy_segments_async([(src, dst, 4096)], done_flag=flags, done_value=9, mode=0, ctas=4)
        gpu.wait_flags(flags, 1, 9, timeout_ms=2000)
        assert gpu.exchange_status() == 0
        assert (gpu.download(dst, 4096) == 0x5A).all()
    finally:
        for p in (src, dst, flags):
            gpu.dev_free(p)


def _rank(rank, world, port, tmpdir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import datetime
    import torch
    import torch.distributed as dist
    from npu_plugin_b200 import workloads as W
    from npu_plugin_b200.const import CudaBackend
    from npu_plugin_b200.sharded import PushTransport, ShardedFolder, blob_digest
    from test_multirank_gloo import _model
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))

    class Comm:
        def all_gather(self, obj):
            out = [None] * world
            dist.all_gather_object(out, obj)
            return out

    gpu = CudaBackend(rank)
    decls = _model()
    sf = ShardedFolder(gpu, decls, rank, world, PushTransport(Comm(), timeout_ms=5000), weights=[0.5, 0.5], nchunks=3)
    mine = [decls[i] for i in sf.layout.mine[rank]]
    ins = [gpu.dev_alloc(d.nbytes) for d in mine]
    side = []
    for d in mine:
        oc = d.base_type.shape[0]
        side.append((gpu.dev_alloc(4 * oc), gpu.dev_alloc(4 * oc)) if W.has_quantizer(d) else None)
    for p, d in zip(ins, mine):
        W.fill_device(gpu, d, p)
    table = None
    for _ in range(3):
        rows = sf.step(ins, side, True)
        if rank == 0:
            table = sf.collect(rows)
            sf.release()
    sf.t.check(sf)
    if rank == 0:
        np.save(os.path.join(tmpdir, "blob.npy"), gpu.download(sf.t.blob_ptr(), sf.layout.blob_bytes))
        np.save(os.path.join(tmpdir, "table.npy"), np.array(table, dtype=np.int64))
        with open(os.path.join(tmpdir, "digest.txt"), "w") as f:
            f.write(blob_digest(gpu, sf.t.blob_ptr(), table))
    dist.barrier()
    sf.close()
    dist.destroy_process_group()


def test_two_gpu_sharded_fold_equals_single_rank_blob(gpu, oracle, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs (ranks that wait on one another must not share a device)")
    import torch.multiprocessing as mp
    from npu_plugin_b200.sharded import combine_digests
    from test_multirank_gloo import _single_rank_reference
    mp.spawn(_rank, args=(2, 29500 + os.getpid() % 2000, str(tmp_path)), nprocs=2, join=True)
    blob, table = np.load(tmp_path / "blob.npy"), np.load(tmp_path / "table.npy").tolist()
    ref_blob, ref_table = _single_rank_reference()  # folded by the CPU oracle
    for (i, off, size, comp), (j, roff, rsize, rcomp) in zip(table, ref_table):
        assert (i, size, bool(comp)) == (j, rsize, bool(rcomp))
        assert np.array_equal(blob[off:off + size], ref_blob[roff:roff + rsize]), f"constant {i}"
    want = combine_digests([oracle.digest64(ref_blob[o:o + s]) for _, o, s, _ in ref_table], ref_table)
    assert open(tmp_path / "digest.txt").read() == want


def test_copy_ordered_behind_a_compression_ticket(gpu, oracle):
    """The two-step in-place compression with a transfer ordered behind its ticket alone: the copy sees the
    finished streams although more work was queued on the context's stream after the compression."""
    import ctypes as C
    from npu_plugin_b200.const import raise_for
    rng = np.random.default_rng(21)
    sizes = [300_000, 64 * 1024, 5000]
    slots = [np.clip(np.rint(rng.laplace(0, 4, n)), -127, 127).astype(np.int8).view(np.uint8) for n in sizes]
    slots[2] = rng.integers(0, 256, sizes[2], dtype=np.uint8)  # does not shrink: stays as it is
    offs = [0, 512 * 600, 512 * 800]
    total = 512 * 900
    buf, mirror, flags, noise = gpu.dev_alloc(total), gpu.dev_alloc(total), gpu.dev_alloc(256), gpu.dev_alloc(1 << 24)
    try:
        for o, x in zip(offs, slots):
            gpu.upload(buf + o, x)
        gpu.fill_zero(mirror, total)
        gpu.fill_zero(flags, 256)
        ptrs = (C.c_void_p * 3)(*[buf + o for o in offs])
        lens = (C.c_size_t * 3)(*sizes)
        ticket = C.c_int()
        raise_for(gpu.lib.b200c_btc_compress_inplace_begin(gpu.ctx, 3, ptrs, lens, C.byref(ticket)), gpu.lib.b200c_last_error())
        # more work behind the compression on the same stream: the transfer must not wait for it to be correct
        gpu.fill_zero(noise, 1 << 24)
        out_sizes, comp = (C.c_size_t * 3)(), (C.c_int32 * 3)()
        raise_for(gpu.lib.b200c_btc_compress_inplace_end(gpu.ctx, ticket.value, out_sizes, comp), gpu.lib.b200c_last_error())
        assert list(comp) == [1, 1, 0] and out_sizes[2] == sizes[2]
        segs = [(buf + o, mirror + o, int(n)) for o, n in zip(offs, out_sizes)]
        gpu.copy_segments_async(segs, done_flag=flags, done_value=3, mode=2, ctas=8, after_ticket=ticket.value)
        gpu.wait_flags(flags, 1, 3, timeout_ms=2000)
        assert gpu.exchange_status() == 0
        got = gpu.download(mirror, total)
        for o, n, x, c in zip(offs, out_sizes, slots, comp):
            live = got[o:o + n]
            if c:
                stream, not_smaller = oracle.btc_compress(x)
                assert not not_smaller and np.array_equal(live, stream)
            else:
                assert np.array_equal(live, x)
        # a ticket is spent once collected; an unknown ticket is an argument error
        assert gpu.lib.b200c_btc_compress_inplace_end(gpu.ctx, ticket.value, out_sizes, comp) == A.ERR_INVALID
    finally:
        for p in (buf, mirror, flags, noise):
            gpu.dev_free(p)
