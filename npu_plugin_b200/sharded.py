"""Whole-model folding sharded over the GPUs of one machine (one process per GPU).

The reference writes all constants of a model into one blob from a parallel loop inside one process
(serializeBinaryData, src/vpux_compiler/src/dialect/VPUIP/graph-schema/export.cpp:453-493).  Here the
constants are partitioned by tensor, every rank folds and compresses its share with no data-path
collective, and the one exchange is the transfer of finished slots into the blob buffer of rank 0.

Layout.  Compression works in place, so the slot layout is known before any data exists: the blob is
the concatenation of every rank's region, a region is the concatenation of that rank's chunks, a chunk
the 512-byte aligned slots of its constants (ShardFolder).  A rank's local buffer mirrors its region
byte for byte; rank 0's region is the head of the blob itself, so its constants are folded where they
stay.

Exchange.  The owner pushes: after a chunk has been folded and compressed, the live bytes of its slots
(and the chunk's rows of the segment table) are copied into rank 0's buffer by the pushing rank's own
copy kernel through a CUDA IPC mapping, and a sequence word per (chunk, rank) in rank 0's memory is
raised.  Rank 0 ends its step with bounded waits on those words and releases the buffer for the next
step through a word in every pusher's memory.  No host message is exchanged per step.

`Transport` is the part that moves bytes; PushTransport is the NVLink form, and the CPU tests run the
same ShardedFolder over a host transport (torch.distributed send/recv on gloo).
"""
import ctypes as C

import numpy as np

from .blob import SEGMENT_ALIGN, ShardFolder, gather_aware_weights, partition


class ExchangeError(RuntimeError):
    """A bounded wait of the exchange ran out: a peer is missing or stuck."""


def split_chunks(indices, nbytes_of, nchunks):
    """Cuts a list of constant indices into at most `nchunks` consecutive groups of about equal bytes."""
    total = sum(nbytes_of(i) for i in indices)
    per = (total + nchunks - 1) // nchunks if indices else 1
    out, cur, cur_bytes = [], [], 0
    for i in indices:
        if cur and cur_bytes + nbytes_of(i) > per and len(out) < nchunks - 1:
            out.append(cur)
            cur, cur_bytes = [], 0
        cur.append(i)
        cur_bytes += nbytes_of(i)
    if cur:
        out.append(cur)
    return out


class Layout:
    """Who owns which constant, how every rank cuts its share into chunks, and where every slot lies in
    the assembled blob.  Pure arithmetic: identical on every rank given the same declarations."""

    TABLE_ROW = 4  # int64 words per constant: index, blob offset, size, compressed flag

    def __init__(self, decls, world, weights=None, nchunks=None, folded_size_of=None, rank0_chunks=1):
        self.world = world
        self.owner = partition(decls, world, weights)
        self.mine = [[i for i, o in enumerate(self.owner) if o == r] for r in range(world)]
        if nchunks is None:
            nchunks = 4
        # rank 0's slots never travel, so with device-resident inputs it has nothing to pipeline: one chunk
        # (host inputs are another matter: its uploads and downloads overlap chunk by chunk)
        self.chunks = [split_chunks(self.mine[r], lambda i: decls[i].nbytes, rank0_chunks if r == 0 else nchunks)
                       for r in range(world)]
        self.nchunks = max(1, max(len(c) for c in self.chunks))
        self.region_off, self.region_bytes, self.chunk_off = [], [], []
        at = 0
        for r in range(world):
            self.region_off.append(at)
            offs, local = [], 0
            for chunk in self.chunks[r]:
                offs.append(local)
                end = 0
                for i in chunk:
                    end = (end + folded_size_of(i) + SEGMENT_ALIGN - 1) // SEGMENT_ALIGN * SEGMENT_ALIGN
                local += end
            self.chunk_off.append(offs)
            self.region_bytes.append(local)
            at += local
        self.blob_bytes = max(at, 1)
        # the segment table follows the blob: one row per constant, grouped like the slots
        self.table_off = (self.blob_bytes + 255) // 256 * 256
        self.table_row_of = {}
        row = 0
        for r in range(world):
            for chunk in self.chunks[r]:
                for i in chunk:
                    self.table_row_of[i] = row
                    row += 1
        self.table_bytes = max(1, row) * self.TABLE_ROW * 8
        self.flags_off = (self.table_off + self.table_bytes + 255) // 256 * 256
        self.flags_bytes = self.nchunks * world * 8
        self.buffer_bytes = self.flags_off + self.flags_bytes


class ShardedFolder:
    """One rank's part of a sharded whole-model fold.

    backend   : the rank's CudaBackend (or a stand-in with the same folding interface for CPU tests)
    decls     : every ConstantDecl of the model, identical on all ranks
    transport : moves finished chunks to rank 0 (PushTransport on GPUs)
    weights   : shares of the work per rank for partition(); default: rank 0's share balances its compute
                against the ingress of everything the other ranks produce (gather_aware_weights with the
                measured rates: about 5 TB/s of algorithmic bytes for the kernels, and 0.54 TB/s of blob bytes
                entering rank 0 while its own kernels keep its memory busy -- the link itself sustains about
                0.62 TB/s then, the rest is the start-up before the first chunk of a step is ready)
    """

    def __init__(self, backend, decls, rank, world, transport, weights=None, nchunks=None, folder_cls=ShardFolder,
                 compute_rate=5.0e12, link_rate=0.54e12, rank0_chunks=1):
        self.b, self.decls, self.rank, self.world, self.t = backend, decls, rank, world, transport
        if weights is None:
            total_in = sum(d.nbytes for d in decls)
            # algorithmic bytes of a constant are about twice its input bytes, its blob bytes about half
            weights = gather_aware_weights(world, compute_seconds=2.0 * total_in / compute_rate,
                                           transfer_seconds=0.5 * total_in / link_rate)
        self.weights = list(weights)
        sizes = {}

        def folded_size_of(i):
            if i not in sizes:
                sizes[i] = backend.infer_type(decls[i].base_type, decls[i].transforms).getTotalAllocSize()
            return sizes[i]

        self.layout = Layout(decls, world, self.weights, nchunks, folded_size_of, rank0_chunks)
        L = self.layout
        self.my_chunks = L.chunks[rank]
        self.folders = [folder_cls(backend, [decls[i] for i in c]) for c in self.my_chunks]
        for k, f in enumerate(self.folders):  # the folders' own slot arithmetic must agree with the layout's
            nxt = L.chunk_off[rank][k + 1] if k + 1 < len(self.folders) else L.region_bytes[rank]
            assert f.folded_bytes <= max(1, nxt - L.chunk_off[rank][k]), "slot layout mismatch"
        # blob offset of every slot of every chunk of this rank
        self._slot_off = [[L.region_off[rank] + L.chunk_off[rank][k] + off for off in f.folded_offsets]
                          for k, f in enumerate(self.folders)]
        self.seq = 0
        self.local_base = transport.setup(self)
        self._rows = np.zeros((max(1, len(L.mine[rank])), Layout.TABLE_ROW), dtype=np.int64)

    # ------------------------------------------------------------------ one step
    def step(self, in_ptrs, side_ptrs=None, data_on_device=True, hooks=None, max_batch_bytes=None):
        """Folds and compresses this rank's constants; peers push every chunk to rank 0 as it completes.
        in_ptrs / side_ptrs are indexed like layout.mine[rank] (concatenated chunks).  Returns this rank's
        rows of the segment table [(constant index, blob offset, size, compressed)].  On rank 0 call
        collect() afterwards to wait for the peers.  hooks(name, k) is called around the phases of chunk k
        (the benchmark records CUDA events there)."""
        L, r = self.layout, self.rank
        self.seq += 1
        self.t.begin_step(self)
        rows, at = [], 0
        pending = None  # (chunk number, ticket) of the compression queued last

        def finish(k, ticket):
            # sizes of chunk k are known once its compression has run: its table rows, and (peers) its push
            size, comp = self.folders[k].compress_inplace_end(ticket)
            chunk_rows = list(zip(self.my_chunks[k], self._slot_off[k], size.tolist(), comp.astype(np.int64).tolist()))
            if r != 0:
                self.t.push_chunk(self, k, chunk_rows, after_ticket=ticket)
            return chunk_rows

        for k, (chunk, f) in enumerate(zip(self.my_chunks, self.folders)):
            n = len(chunk)
            base = self.local_base + L.chunk_off[r][k]
            if hooks:
                hooks("fold0", k)
            f.fold(in_ptrs[at:at + n], base, data_on_device, side_ptrs[at:at + n] if side_ptrs is not None else None,
                   max_batch_bytes=max_batch_bytes)
            if hooks:
                hooks("fold1", k)
            if hasattr(f, "compress_inplace_begin") and r == 0:
                # The compression of chunk k is only queued here; the host goes on to plan the fold of chunk
                # k + 1 while the device compresses, and reads the sizes of chunk k after that.  Only the
                # assembling rank works this way: a pushing rank sends chunk k the moment it is complete, and
                # measured on four GPUs its pushes arrived later when the next chunk's kernels were already
                # queued behind them (4.8 ms per step instead of 3.9).
                ticket = f.compress_inplace_begin(base)
                if hooks:
                    hooks("codec1", k)  # on the stream: right behind the chunk's compression
                if pending is not None:
                    rows += finish(*pending)
                pending = (k, ticket)
            else:
                segs = f.compress_inplace(base)  # synchronises: the chunk is complete
                if hooks:
                    hooks("codec1", k)
                chunk_rows = [(chunk[j], L.region_off[r] + L.chunk_off[r][k] + off, size, int(comp)) for j, off, size, comp in segs]
                if r != 0:
                    self.t.push_chunk(self, k, chunk_rows)
                rows += chunk_rows
            at += n
        if pending is not None:
            rows += finish(*pending)
        if r != 0:
            self.t.finish_step(self, len(self.folders))
        return rows

    def chunk_span(self, r, k):
        """(blob offset, bytes) of chunk k of rank r."""
        L = self.layout
        lo = L.chunk_off[r][k]
        hi = L.chunk_off[r][k + 1] if k + 1 < len(L.chunk_off[r]) else L.region_bytes[r]
        return L.region_off[r] + lo, hi - lo

    def download_chunk(self, host_ptr, k, own=True):
        """Rank 0: queues, on the transfer stream, the copy of chunk k of every rank into (pinned) host memory
        at the blob's own offsets -- rank 0's chunk k as soon as the context's stream has produced it, the
        peers' chunk k behind a bounded wait for their flags.  The context's stream is never held back, so
        early chunks cross PCIe while later ones are still being folded or still arrive over NVLink.
        Returns the bytes queued."""
        assert self.rank == 0
        L, blob, total = self.layout, self.t.blob_ptr(), 0
        if own and k < len(L.chunks[0]):
            off, n = self.chunk_span(0, k)
            self.b.copy_segments_async([(blob + off, host_ptr + off, n)], mode=1)
            total += n
        segs = []
        for r in range(1, self.world):
            if k < len(L.chunks[r]):
                off, n = self.chunk_span(r, k)
                segs.append((blob + off, host_ptr + off, n))
                total += n
        if segs:
            self.t.wait_chunk(self, k, on_transfer_stream=True)
            self.b.copy_segments_async(segs, mode=1)
        return total

    def download(self, host_ptr, first_chunk=0):
        """Rank 0: download_chunk for every chunk from first_chunk on.  Follow with collect()."""
        return sum(self.download_chunk(host_ptr, k) for k in range(first_chunk, self.layout.nchunks))

    def collect(self, own_rows):
        """Rank 0: waits (bounded) until every peer's chunks of this step have arrived and returns the full
        segment table, one (constant index, blob offset, size, compressed) per constant in model order.
        Raises ExchangeError when a wait runs out."""
        assert self.rank == 0
        rows = list(own_rows) + self.t.collect(self)
        rows.sort()  # by constant index
        n = len(self.decls)
        if len(rows) != n or rows[0][0] != 0 or rows[-1][0] != n - 1 or \
                (self.world > 1 and [x[0] for x in rows] != list(range(n))):
            raise ExchangeError("the gathered segment table does not cover every constant exactly once")
        return rows

    def release(self):
        """Rank 0: the blob of this step has been consumed; the peers may write the next one."""
        self.t.release(self)

    def close(self):
        self.t.close(self)


class PushTransport:
    """NVLink transport: CUDA IPC windows + the library's copy kernel (b200c_copy_segments_async).

    comm supplies the host-side set-up exchange: comm.all_gather(obj) -> list of every rank's object
    (torch.distributed.all_gather_object on a gloo group in the benchmark).  Nothing else goes through
    the host."""

    def __init__(self, comm, timeout_ms=10000, mode=0, ctas=64):
        self.comm, self.timeout_ms, self.mode, self.ctas = comm, timeout_ms, mode, ctas
        self.buffer = self.release_word = self.mapped_blob = self.rows_host = None
        self.mapped_release = []

    def setup(self, sf):
        b, L, rank = sf.b, sf.layout, sf.rank
        if rank == 0:
            # zeroed once, like the buffers the reference's writers pre-zero (export.cpp:471-473): bytes no
            # constant ever writes (slot padding, the tail behind a short Sparsify result) stay zero
            self.buffer = b.dev_alloc(L.buffer_bytes)
            b.fill_zero(self.buffer, L.buffer_bytes)
            desc = b.ipc_export(self.buffer, L.buffer_bytes)
        else:
            # local mirror of this rank's region, then the release word rank 0 writes
            self.local_bytes = (max(1, L.region_bytes[rank]) + 255) // 256 * 256
            self.buffer = b.dev_alloc(self.local_bytes + 256)
            self.release_word = self.buffer + self.local_bytes
            b.fill_zero(self.buffer, self.local_bytes + 256)
            desc = b.ipc_export(self.release_word, 8)
            n_rows = max(1, len(L.mine[rank]))
            self.rows_host = b.pinned_alloc(n_rows * Layout.TABLE_ROW * 8)
            self.rows_np = np.ctypeslib.as_array((C.c_int64 * (n_rows * Layout.TABLE_ROW)).from_address(self.rows_host))
        descs = self.comm.all_gather(desc)
        if rank == 0:
            self.mapped_release = [b.ipc_open(d) for d in descs[1:]]
        else:
            self.mapped_blob = b.ipc_open(descs[0])
        self.comm.all_gather(None)  # every window is open before anyone stores through one
        return self.buffer

    def blob_ptr(self):
        return self.buffer

    def begin_step(self, sf):
        if sf.rank != 0:
            # the local slots are about to be overwritten: the pushes of the previous step must have read them
            sf.b.stream_join()
            self._row_at = 0

    def push_chunk(self, sf, k, chunk_rows, after_ticket=None):
        b, L, rank = sf.b, sf.layout, sf.rank
        region = L.region_off[rank]
        segs = [(self.buffer + (off - region), self.mapped_blob + off, size) for _, off, size, _ in chunk_rows]
        # the chunk's table rows travel with it (pinned host memory is readable by the copy kernel)
        n = len(chunk_rows)
        if n:
            first_row = L.table_row_of[chunk_rows[0][0]]
            a = self._row_at * Layout.TABLE_ROW
            self.rows_np[a:a + n * Layout.TABLE_ROW] = np.asarray(chunk_rows, dtype=np.int64).reshape(-1)
            segs.append((self.rows_host + a * 8, self.mapped_blob + L.table_off + first_row * Layout.TABLE_ROW * 8,
                         n * Layout.TABLE_ROW * 8))
            self._row_at += n
        flag = self.mapped_blob + L.flags_off + (k * L.world + rank) * 8
        b.copy_segments_async(segs, wait_flag=self.release_word if k == 0 else None, wait_value=sf.seq - 1,
                              done_flag=flag, done_value=sf.seq, timeout_ms=self.timeout_ms, mode=self.mode, ctas=self.ctas,
                              after_ticket=after_ticket)

    def finish_step(self, sf, chunks_done):
        # chunks this rank does not have still owe their flag (the first of them waits for the release when
        # the rank has no chunk at all)
        b, L, rank = sf.b, sf.layout, sf.rank
        for kk in range(chunks_done, L.nchunks):
            b.copy_segments_async([], wait_flag=self.release_word if kk == 0 else None, wait_value=sf.seq - 1,
                                  done_flag=self.mapped_blob + L.flags_off + (kk * L.world + rank) * 8, done_value=sf.seq,
                                  timeout_ms=self.timeout_ms, mode=0, ctas=1)

    def check(self, sf):
        """Waits for this rank's queued work and raises if one of its bounded waits ran out."""
        status = sf.b.exchange_status()
        if status:
            raise ExchangeError(f"exchange timed out on rank {sf.rank} (status {status})")

    def wait_chunk(self, sf, k, on_transfer_stream=False):
        """Rank 0: queue the bounded wait for chunk k of every peer on the context's stream (or on its transfer
        stream, where it holds back only the downloads queued after it)."""
        L = sf.layout
        if L.world > 1:
            sf.b.wait_flags(self.buffer + L.flags_off + (k * L.world + 1) * 8, L.world - 1, sf.seq, self.timeout_ms,
                            on_transfer_stream)

    def collect(self, sf):
        b, L = sf.b, sf.layout
        for k in range(L.nchunks):
            self.wait_chunk(sf, k)
        status = b.exchange_status()  # waits for the stream
        if status:
            raise ExchangeError(f"exchange timed out (status {status}): a peer did not deliver its chunks within "
                                f"{self.timeout_ms} ms")
        n_own = len(L.mine[0])
        n_all = len(sf.decls)
        if n_all == n_own:
            return []
        raw = b.download(self.buffer + L.table_off + n_own * Layout.TABLE_ROW * 8, (n_all - n_own) * Layout.TABLE_ROW * 8)
        t = raw.view(np.int64).reshape(-1, Layout.TABLE_ROW)
        return [tuple(int(v) for v in row) for row in t]

    def release(self, sf):
        if sf.rank == 0 and self.mapped_release:
            sf.b.signal_flags(self.mapped_release, sf.seq)

    def close(self, sf):
        b = sf.b
        try:
            b.synchronize()
        except Exception:
            pass
        for m in self.mapped_release:
            b.ipc_close(m)
        if self.mapped_blob:
            b.ipc_close(self.mapped_blob)
        self.mapped_release, self.mapped_blob = [], None
        try:
            self.comm.all_gather(None)  # nobody frees memory another rank still has mapped
        except Exception:
            pass
        b.dev_free(self.buffer)
        b.pinned_free(self.rows_host)
        self.buffer = self.rows_host = None


class SingleTransport:
    """One rank: the blob is a plain device buffer and nothing travels."""

    def __init__(self):
        self.buffer = None

    def setup(self, sf):
        self.buffer = sf.b.dev_alloc(sf.layout.buffer_bytes)
        sf.b.fill_zero(self.buffer, sf.layout.buffer_bytes)
        return self.buffer

    def blob_ptr(self):
        return self.buffer

    def begin_step(self, sf):
        pass

    def push_chunk(self, sf, k, chunk_rows):
        raise AssertionError("a single rank has nothing to push")

    def finish_step(self, sf, chunks_done):
        pass

    def wait_chunk(self, sf, k, on_transfer_stream=False):
        pass

    def check(self, sf):
        pass

    def collect(self, sf):
        return []

    def release(self, sf):
        pass

    def close(self, sf):
        sf.b.dev_free(self.buffer)
        self.buffer = None


def tensor_log_lines(decls, table, folded_size_of=None):
    """One JSON line per constant of an assembled blob, in model order: name, transformation names, bytes in,
    bytes stored in the blob, compressed flag and ratio -- the counterpart of the reference's per-constant trace
    lines (the transformation trace of content.cpp:188, the compression ratio of compress_weights_btc.cpp:193-196)."""
    import json
    out = []
    for (i, off, size, comp), d in zip(table, decls):
        rec = {"constant": d.name, "transformations": [t.getTransformationName() for t in d.transforms],
               "bytes_in": int(d.nbytes), "blob_offset": int(off), "bytes_stored": int(size), "compressed": bool(comp)}
        if folded_size_of is not None:
            folded = int(folded_size_of(i))
            rec["bytes_folded"] = folded
            rec["ratio"] = round(size / folded, 4) if folded else None
        out.append(json.dumps(rec))
    return out


def blob_digest(backend, blob_ptr, table):
    """Digest of an assembled blob that does not depend on where the slots lie: the per-constant digests of
    the live bytes (b200c_digest64_batch), combined in model order with size and compressed flag."""
    ptrs = [blob_ptr + off for _, off, _, _ in table]
    sizes = [size for _, _, size, _ in table]
    return combine_digests(backend.digest64(ptrs, sizes), table)


def combine_digests(digests, table):
    mask = (1 << 64) - 1

    def mix(x):
        x ^= x >> 30
        x = (x * 0xBF58476D1CE4E5B9) & mask
        x ^= x >> 27
        x = (x * 0x94D049BB133111EB) & mask
        return x ^ (x >> 31)

    h = 0
    for d, (idx, _, size, comp) in zip(digests, table):
        h = mix(h ^ d ^ ((size << 1 | int(bool(comp))) * 0x9E3779B97F4A7C15 & mask) ^ (idx + 1))
    return f"{h:016x}"
