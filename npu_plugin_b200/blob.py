"""Whole-model constant folding: the B200 counterpart of the reference's blob constant writer.

The reference serialises a model's constants with a parallel loop over every Const::DeclareOp --
fold(), then copyTo() into an 8-byte aligned buffer (serializeBinaryData,
src/vpux_compiler/src/dialect/VPUIP/graph-schema/export.cpp:453-493) -- after the weight compression
pass replaced compressible ones (src/vpux_compiler/src/dialect/VPUIP/passes/compress_weights_btc.cpp:64-72,
120-136).  Here the declarations of one rank's shard are folded back to back on the device into one
"folded" arena and then compressed in one batched call; segments that do not shrink, or are below
the 4 KB gate, stay uncompressed, as the reference leaves them.

Descriptors are marshalled once (prepare) so that a step is only C ABI calls.
"""
import ctypes as C

import numpy as np

from . import _cabi as A
from .const import NDType, chain_to_c, out_type_slot, raise_for

MIN_COMPRESS_BYTES = 4096  # MIN_INPUT_SIZE = 4_KB, compress_weights_btc.cpp:120-125
SEGMENT_ALIGN = 512        # folded segments start on a swizzle-block boundary (>= the 8 bytes of export.cpp:473-476)


class ConstantDecl:
    """One constant: base content (pointer + byte size + type) and its transformation list."""

    def __init__(self, name, base_type, transforms, nbytes, compress=True, is_splat=False):
        self.name, self.base_type, self.transforms = name, base_type, list(transforms)
        self.nbytes, self.compress, self.is_splat = int(nbytes), bool(compress), bool(is_splat)


def partition(decls, world_size, weights=None):
    """Deterministic longest-processing-time assignment of constants to ranks by input bytes.
    `weights` (one positive number per rank, default all equal) are the shares of the work the ranks
    should get: a rank with twice the weight ends up with about twice the bytes."""
    w = [1.0] * world_size if weights is None else [float(x) for x in weights]
    if len(w) != world_size or min(w) <= 0:
        raise ValueError("weights: one positive number per rank")
    order = sorted(range(len(decls)), key=lambda i: (-decls[i].nbytes, i))
    load = [0] * world_size
    owner = [0] * len(decls)
    for i in order:
        r = min(range(world_size), key=lambda k: ((load[k] + decls[i].nbytes) / w[k], k))
        owner[i] = r
        load[r] += decls[i].nbytes
    return owner


def gather_aware_weights(world_size, compute_seconds, transfer_seconds):
    """Shares for partition() when every other rank's output must travel to rank 0: rank 0's share f
    balances its own compute time f * compute against the ingress time (1 - f) * transfer of what the
    others produce, and never drops below an equal split.  compute_seconds: one GPU doing the whole
    job; transfer_seconds: the whole output crossing one link."""
    if world_size == 1:
        return [1.0]
    f = max(1.0 / world_size, transfer_seconds / (compute_seconds + transfer_seconds))
    f = min(f, 0.95)
    return [f] + [(1.0 - f) / (world_size - 1)] * (world_size - 1)


class ShardFolder:
    """Folds and compresses the constants one rank owns.  All buffers are caller-provided device
    (or pinned host) memory; nothing is allocated per step."""

    def __init__(self, backend, decls):
        self.b, self.lib, self.ctx = backend, backend.lib, backend.ctx
        self.decls = decls
        self._keep = []
        self._prepared = []
        self._marshalled = None
        self._group_cache = {}
        self.folded_offsets, self.folded_sizes = [], []
        at = 0
        for d in decls:
            final = backend.infer_type(d.base_type, d.transforms)
            size = final.getTotalAllocSize()
            bt = d.base_type.to_c(self._keep)
            ch = chain_to_c(d.transforms, self._keep)
            ot = out_type_slot(1, self._keep)
            self._prepared.append((bt, ch, len(d.transforms), ot))
            self.folded_offsets.append(at)
            self.folded_sizes.append(size)
            at = (at + size + SEGMENT_ALIGN - 1) // SEGMENT_ALIGN * SEGMENT_ALIGN
        self.folded_bytes = max(at, 1)
        n = max(1, len(decls))
        self._in_ptrs = (C.c_void_p * n)()
        self._sizes = (C.c_size_t * n)()
        self._out_off = (C.c_size_t * n)()
        self._out_size = (C.c_size_t * n)()
        self._not_smaller = (C.c_int32 * n)()
        self._nb = C.c_size_t()
        self._items = (A.b200c_fold_item * n)()
        for i, (bt, ch, k, ot) in enumerate(self._prepared):
            it = self._items[i]
            it.base = C.pointer(bt)
            it.nbytes = decls[i].nbytes
            it.is_splat = int(decls[i].is_splat)
            it.n = k
            it.chain = C.cast(ch, C.POINTER(A.b200c_xform))
            it.out_cap = self.folded_sizes[i]
        self.comp_idx = [i for i, d in enumerate(decls) if d.compress and self.folded_sizes[i] >= MIN_COMPRESS_BYTES]
        # array views of the call arguments, so that a step costs no Python loop over the constants
        self._in_ptrs_np = np.ctypeslib.as_array(C.cast(self._in_ptrs, C.POINTER(C.c_uint64)), (n,))
        self._sizes_np = np.ctypeslib.as_array(C.cast(self._sizes, C.POINTER(C.c_uint64)), (n,))
        self._out_size_np = np.ctypeslib.as_array(C.cast(self._out_size, C.POINTER(C.c_uint64)), (n,))
        self._flag_np = np.ctypeslib.as_array(self._not_smaller)
        self._comp_idx_np = np.asarray(self.comp_idx, dtype=np.int64)
        self._offsets_np = np.asarray(self.folded_offsets, dtype=np.int64)
        self._folded_sizes_np = np.asarray(self.folded_sizes, dtype=np.int64)
        self._comp_marshalled = None
        self.blob_bound = sum((backend.btc_bound(self.folded_sizes[i]) + 31) // 32 * 32 for i in self.comp_idx) + 64

    def fold(self, data_ptrs, folded_ptr, data_on_device=True, side_ptrs=None, max_batch_bytes=None):
        """fold() + copyTo() of every constant into folded_ptr + folded_offsets[i] through the batched
        entry point (asynchronous; errors surface at the next synchronising call).  With host input
        the items are issued in groups of at most max_batch_bytes so the staging memory stays bounded."""
        lib, ctx = self.lib, self.ctx
        n = len(self.decls)
        key = (tuple(data_ptrs), folded_ptr, tuple(side_ptrs) if side_ptrs is not None else None)
        if key != self._marshalled:  # the same buffers as last time: the item array is already filled in
            for i in range(n):
                it = self._items[i]
                it.data = data_ptrs[i]
                it.out = folded_ptr + self.folded_offsets[i]
                if side_ptrs is not None and side_ptrs[i] is not None:
                    ch = self._prepared[i][1]
                    for k in range(self._prepared[i][2]):
                        if ch[k].kind == A.X_QUANTIZE_SYNTH:
                            ch[k].side0, ch[k].side1 = side_ptrs[i]
            self._marshalled = key
        for first, last in self._groups(max_batch_bytes):
            at = C.cast(C.addressof(self._items) + first * C.sizeof(A.b200c_fold_item), C.POINTER(A.b200c_fold_item))
            rc = lib.b200c_fold_batch(ctx, at, last - first, int(data_on_device), 1, A.FOLD_ASYNC)
            if rc != A.OK:
                raise_for(rc, lib.b200c_last_error())

    def _groups(self, max_batch_bytes):
        """[first, last) ranges of consecutive constants whose input bytes stay within max_batch_bytes (one range
        for all of them without a limit; a constant above the limit goes alone).  Worked out once per limit: a
        step must not pay a Python loop over the constants."""
        if max_batch_bytes not in self._group_cache:
            n, out, first = len(self.decls), [], 0
            while first < n:
                last, total = first, 0
                while last < n and (last == first or max_batch_bytes is None or total + self.decls[last].nbytes <= max_batch_bytes):
                    total += self.decls[last].nbytes
                    last += 1
                out.append((first, last))
                first = last
            self._group_cache[max_batch_bytes] = out
        return self._group_cache[max_batch_bytes]

    def written_sizes(self):
        """Bytes the last fold() wrote per constant.  Equal to folded_sizes except for contents that are shorter
        than their type says (Sparsify without numActualElements: the values end where the data decides, the
        rest of the pre-zeroed slot is never touched)."""
        return [int(self._items[i].out_bytes) for i in range(len(self.decls))]

    def fold_one_by_one(self, data_ptrs, folded_ptr, data_on_device=True, side_ptrs=None):
        """Same result through one b200c_fold call per constant."""
        lib, ctx = self.lib, self.ctx
        flags = A.FOLD_ASYNC
        for i, (bt, ch, n, ot) in enumerate(self._prepared):
            d = self.decls[i]
            self._marshalled = None
            if side_ptrs is not None and side_ptrs[i] is not None:
                for k in range(n):
                    if ch[k].kind == A.X_QUANTIZE_SYNTH:
                        ch[k].side0, ch[k].side1 = side_ptrs[i]
            rc = lib.b200c_fold(ctx, C.byref(bt), data_ptrs[i], d.nbytes, int(d.is_splat), int(data_on_device), ch, n,
                                folded_ptr + self.folded_offsets[i], self.folded_sizes[i], 1, C.byref(self._nb), None,
                                flags)
            if rc != A.OK:
                raise_for(rc, lib.b200c_last_error())

    def compress(self, folded_ptr, blob_ptr, blob_cap):
        """Batched block compression of the folded segments into blob_ptr.  Returns a list of
        (decl index, blob offset, size, compressed flag); synchronises."""
        k = len(self.comp_idx)
        if k == 0:
            raise_for(self.lib.b200c_synchronize(self.ctx), self.lib.b200c_last_error())
            return []
        self._comp_marshalled = None
        for j, i in enumerate(self.comp_idx):
            self._in_ptrs[j] = folded_ptr + self.folded_offsets[i]
            self._sizes[j] = self.folded_sizes[i]
        rc = self.lib.b200c_btc_compress_batch(self.ctx, k, self._in_ptrs, self._sizes, blob_ptr, blob_cap,
                                               self._out_off, self._out_size, self._not_smaller)
        raise_for(rc, self.lib.b200c_last_error())
        return [(i, self._out_off[j], self._out_size[j], not self._not_smaller[j]) for j, i in enumerate(self.comp_idx)]

    def compress_inplace(self, folded_ptr):
        """Compresses every eligible folded segment where it lies: a segment that shrinks is replaced
        by its stream (at the same offset), the others stay as they are.  The folded buffer then IS
        the blob.  Returns (decl index, offset, size, compressed flag) for every constant; synchronises."""
        size, flag = self.compress_inplace_arrays(folded_ptr)
        return list(zip(range(len(self.decls)), self.folded_offsets, size.tolist(), flag.tolist()))

    def compress_inplace_begin(self, folded_ptr):
        """First half of compress_inplace_arrays: queues the compression of this folder's slots and returns a
        ticket at once, so that the caller can prepare the next group of constants while the device works.
        Returns None when nothing is eligible."""
        k = len(self.comp_idx)
        if not k:
            return None
        self._marshal_compress(folded_ptr)
        ticket = C.c_int()
        rc = self.lib.b200c_btc_compress_inplace_begin(self.ctx, k, self._in_ptrs, self._sizes, C.byref(ticket))
        raise_for(rc, self.lib.b200c_last_error())
        return ticket.value

    def compress_inplace_end(self, ticket):
        """Second half: waits for the ticket's work only and returns (live sizes, compressed flags)."""
        size = self._folded_sizes_np.copy()
        flag = np.zeros(len(self.decls), dtype=bool)
        if ticket is None:
            return size, flag
        k = len(self.comp_idx)
        rc = self.lib.b200c_btc_compress_inplace_end(self.ctx, ticket, self._out_size, self._not_smaller)
        raise_for(rc, self.lib.b200c_last_error())
        size[self._comp_idx_np] = self._out_size_np[:k].astype(np.int64)
        flag[self._comp_idx_np] = self._flag_np[:k] != 0
        return size, flag

    def _marshal_compress(self, folded_ptr):
        if self._comp_marshalled != folded_ptr:  # the same buffer as last time: the arrays are already filled in
            k = len(self.comp_idx)
            self._in_ptrs_np[:k] = (self._offsets_np[self._comp_idx_np] + folded_ptr).astype(np.uint64)
            self._sizes_np[:k] = self._folded_sizes_np[self._comp_idx_np].astype(np.uint64)
            self._comp_marshalled = folded_ptr

    def compress_inplace_arrays(self, folded_ptr):
        """compress_inplace with the result as two arrays indexed like the constants: (live size in bytes,
        compressed flag)."""
        k = len(self.comp_idx)
        size = self._folded_sizes_np.copy()
        flag = np.zeros(len(self.decls), dtype=bool)
        if k:
            self._marshal_compress(folded_ptr)
            rc = self.lib.b200c_btc_compress_inplace_batch(self.ctx, k, self._in_ptrs, self._sizes, self._out_size,
                                                           self._not_smaller)
            raise_for(rc, self.lib.b200c_last_error())
            size[self._comp_idx_np] = self._out_size_np[:k].astype(np.int64)
            flag[self._comp_idx_np] = self._flag_np[:k] != 0
        else:
            raise_for(self.lib.b200c_synchronize(self.ctx), self.lib.b200c_last_error())
        return size, flag
