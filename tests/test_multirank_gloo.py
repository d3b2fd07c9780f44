"""The multi-rank whole-model fold on CPU ranks (gloo, world sizes 2, 3 and 8).

The routine under test is npu_plugin_b200.sharded.ShardedFolder -- the same partition, chunking, slot
layout, segment table and step/collect/release sequence the benchmark runs on GPUs.  Only the two parts
that need a device are replaced: the per-chunk folder (OracleShardFolder: folding and compression by the
CPU oracle) and the transport (HostTransport below: torch.distributed send/recv instead of stores through
a CUDA IPC window).  The assembled blob must hold, per constant, exactly the bytes a single rank
produces.  A second test lets a rank leave between steps: rank 0 must get an ExchangeError inside the
time limit instead of hanging.
"""
import datetime
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _model():
    """A small model with the benchmark's kinds of constants: quantised linears (incompressible), a
    compressible int8 constant, pass-through f16 constants."""
    sys.path.insert(0, ROOT)
    from npu_plugin_b200 import _cabi as A
    from npu_plugin_b200.blob import ConstantDecl
    from npu_plugin_b200.const import DimsOrder, NDType, Transform, UniformQuantizedPerAxisType
    decls = []

    def linear(o, i):
        q = UniformQuantizedPerAxisType(A.SI8, A.F16, [1.0] * o, [0] * o, 0, -127, 127)
        chain = [Transform(A.X_QUANTIZE_SYNTH, i0=A.QSYNTH_SYM_I8), Transform(A.X_CONVERT_ELEM_TYPE, elem=A.SI8),
                 Transform(A.X_QUANT_CAST, elem=q), Transform(A.X_REORDER, a=DimsOrder.NHWC),
                 Transform(A.X_SWIZZLE_CONSTANT, i0=5, i1=3)]
        d = ConstantDecl(f"w{len(decls)}", NDType((o, i, 1, 1), A.F16), chain, o * i * 2, compress=True)
        d.synth, d.stream = (A.F16, 0, 0.02, 0.0), len(decls)
        decls.append(d)

    for o, i in ((64, 256), (48, 1024), (16, 4096), (40, 1100), (128, 64), (96, 512), (33, 100), (72, 256)):
        linear(o, i)
    qs = UniformQuantizedPerAxisType(A.SI8, A.F16, [1.0] * 64, [0] * 64, 0, -127, 127)
    d = ConstantDecl("small", NDType((64, 1024, 1, 1), A.SI8),
                     [Transform(A.X_QUANT_CAST, elem=qs), Transform(A.X_REORDER, a=DimsOrder.NHWC)], 64 * 1024, compress=True)
    d.synth, d.stream = (A.SI8, 2, 3.0, 0.3), len(decls)
    decls.append(d)
    for n in (512, 4096, 300):
        d = ConstantDecl(f"gain{len(decls)}", NDType((n,), A.F16), [], 2 * n, compress=False)
        d.synth, d.stream = (A.F16, 0, 1.0, 0.0), len(decls)
        decls.append(d)
    return decls


class HostTransport:
    """CPU transport with the interface of npu_plugin_b200.sharded.PushTransport: buffers are numpy
    arrays, a pushed chunk is one send of its table rows and one of its slot bytes."""

    def __init__(self, dist, group):
        self.dist, self.group = dist, group

    def setup(self, sf):
        L = sf.layout
        n = L.buffer_bytes if sf.rank == 0 else max(1, L.region_bytes[sf.rank])
        self.buf = np.zeros(n, np.uint8)
        return self.buf.ctypes.data

    def blob_ptr(self):
        return self.buf.ctypes.data

    def begin_step(self, sf):
        pass

    def push_chunk(self, sf, k, chunk_rows):
        import torch
        L, r = sf.layout, sf.rank
        rows = torch.tensor(chunk_rows, dtype=torch.int64).reshape(-1)
        self.dist.send(rows, dst=0, group=self.group)
        off, n = sf.chunk_span(r, k)
        lo = off - L.region_off[r]
        self.dist.send(torch.from_numpy(self.buf[lo:lo + n]), dst=0, group=self.group)

    def finish_step(self, sf, chunks_done):
        pass

    def wait_chunk(self, sf, k):
        pass

    def collect(self, sf):
        import torch
        from npu_plugin_b200.sharded import ExchangeError, Layout
        L, rows = sf.layout, []
        try:
            for r in range(1, sf.world):
                for k, chunk in enumerate(L.chunks[r]):
                    t = torch.zeros(len(chunk) * Layout.TABLE_ROW, dtype=torch.int64)
                    self.dist.recv(t, src=r, group=self.group)
                    rows += [tuple(int(v) for v in row) for row in t.reshape(-1, Layout.TABLE_ROW)]
                    off, n = sf.chunk_span(r, k)
                    self.dist.recv(torch.from_numpy(self.buf[off:off + n]), src=r, group=self.group)
        except RuntimeError as e:  # gloo: the peer is gone or the time limit passed
            raise ExchangeError(f"a peer did not deliver its chunks: {e}") from e
        return rows

    def release(self, sf):
        pass

    def check(self, sf):
        pass

    def close(self, sf):
        pass


def _fold_rank(rank, world, decls, dist, group, steps, leave_after=None, nchunks=3):
    from oracle_backend import OracleBackend, OracleShardFolder
    from npu_plugin_b200.sharded import ShardedFolder
    from npu_plugin_b200.workloads import SEED
    orc = OracleBackend()
    weights = [0.5] + [0.5 / (world - 1)] * (world - 1) if world > 1 else None
    sf = ShardedFolder(orc, decls, rank, world, HostTransport(dist, group), weights=weights, nchunks=nchunks,
                       folder_cls=OracleShardFolder)
    mine = sf.layout.mine[rank]
    data = [orc.synth_of(decls[i], SEED) for i in mine]
    table = None
    for s in range(steps):
        if leave_after is not None and rank != 0 and s == leave_after:
            return sf, None  # this rank leaves between two steps, nothing of it in flight
        rows = sf.step([x.ctypes.data for x in data], None)
        if rank == 0:
            table = sf.collect(rows)
            sf.release()
    return sf, table


def _worker(rank, world, port, tmpdir, leave_after):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    from npu_plugin_b200.sharded import ExchangeError
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    decls = _model()
    try:
        if leave_after is None:
            sf, table = _fold_rank(rank, world, decls, dist, None, steps=2)
            np.save(os.path.join(tmpdir, f"owner{rank}.npy"), np.array(sf.layout.owner))
            if rank == 0:
                np.save(os.path.join(tmpdir, "blob.npy"), sf.t.buf[:sf.layout.blob_bytes])
                np.save(os.path.join(tmpdir, "table.npy"), np.array(table, dtype=np.int64))
        else:
            import time
            t0 = time.time()
            try:
                _fold_rank(rank, world, decls, dist, None, steps=3, leave_after=leave_after)
                outcome = "finished"
            except ExchangeError:
                outcome = "exchange-error"
            if rank == 0:
                with open(os.path.join(tmpdir, "outcome.txt"), "w") as f:
                    f.write(f"{outcome} {time.time() - t0:.1f}")
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _single_rank_reference():
    """The same model folded by one rank (no exchange at all)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))

    class NoDist:
        pass

    sf, table = _fold_rank(0, 1, _model(), NoDist(), None, steps=1)
    return sf.t.buf[:sf.layout.blob_bytes].copy(), table


@pytest.mark.parametrize("world", [2, 3, 8])
def test_sharded_fold_assembles_the_single_rank_blob(tmp_path, world):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000) + world
    mp.spawn(_worker, args=(world, port, str(tmp_path), None), nprocs=world, join=True)
    owners = [np.load(tmp_path / f"owner{r}.npy") for r in range(world)]
    for o in owners[1:]:
        assert np.array_equal(owners[0], o), "ranks disagree on the partition"
    assert set(owners[0].tolist()) == set(range(world)), "every rank owns something"
    blob, table = np.load(tmp_path / "blob.npy"), np.load(tmp_path / "table.npy")
    ref_blob, ref_table = _single_rank_reference()
    assert [int(r[0]) for r in table] == list(range(len(ref_table)))
    some_compressed = False
    for (i, off, size, comp), (j, roff, rsize, rcomp) in zip(table.tolist(), ref_table):
        assert (i, size, comp) == (j, rsize, rcomp), f"constant {i}: size or compression differs from the single-rank fold"
        assert np.array_equal(blob[off:off + size], ref_blob[roff:roff + rsize]), f"constant {i}: bytes differ"
        some_compressed |= bool(comp)
    assert some_compressed, "the model should hold a constant that compresses"
    # the layout-independent digest the benchmark prints agrees too
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_backend import OracleBackend
    from npu_plugin_b200.sharded import combine_digests
    orc = OracleBackend()
    a = combine_digests([orc.digest64(blob[o:o + s]) for _, o, s, _ in table.tolist()], table.tolist())
    b = combine_digests([orc.digest64(ref_blob[o:o + s]) for _, o, s, _ in ref_table], ref_table)
    assert a == b


def test_rank_leaving_between_steps_gives_an_error_not_a_hang(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000) + 17
    mp.spawn(_worker, args=(2, port, str(tmp_path), 1), nprocs=2, join=True)
    outcome, seconds = open(tmp_path / "outcome.txt").read().split()
    assert outcome == "exchange-error"
    assert float(seconds) < 30.0


def test_tensor_log_lines_describe_every_constant():
    import json
    from npu_plugin_b200.sharded import tensor_log_lines
    decls = _model()
    table = [(i, 512 * i, max(1, d.nbytes // 2), i % 2) for i, d in enumerate(decls)]
    lines = tensor_log_lines(decls, table, lambda i: decls[i].nbytes)
    assert len(lines) == len(decls)
    first = json.loads(lines[0])
    assert first["constant"] == decls[0].name and first["bytes_in"] == decls[0].nbytes
    assert first["bytes_stored"] == table[0][2] and first["compressed"] is False
    assert json.loads(lines[1])["compressed"] is True and 0 < json.loads(lines[1])["ratio"] <= 1
