"""The slot layout of the sharded whole-model fold at the benchmark's world sizes (1, 2, 4, 8), on the
benchmark's own declarations.  Pure host arithmetic: the library's type inference sizes the slots, nothing
is folded.  What a wrong layout would cost on GPUs is a push into another rank's slots, so the checks are
the ones that rule that out: every constant has exactly one owner and one slot, regions and chunks tile the
blob without overlap, the segment table and the sequence words lie behind the blob, and every rank derives
the same layout."""
import numpy as np
import pytest

from npu_plugin_b200 import workloads as W
from npu_plugin_b200.blob import SEGMENT_ALIGN
from npu_plugin_b200.sharded import Layout, ShardedFolder

from test_abi_and_host import HostOnly


class SlotsOnly:
    """Slot arithmetic of a chunk folder, nothing else (the interface ShardedFolder's constructor reads)."""

    def __init__(self, backend, decls):
        self.folded_offsets, at = [], 0
        for d in decls:
            self.folded_offsets.append(at)
            size = backend.infer_type(d.base_type, d.transforms).getTotalAllocSize()
            at = (at + size + SEGMENT_ALIGN - 1) // SEGMENT_ALIGN * SEGMENT_ALIGN
        self.folded_bytes = max(at, 1)


class CachedHost:
    """Type inference through the library, remembered per (base type, chain) object pair: the same
    declarations are sized once however many ranks and world sizes ask."""

    def __init__(self):
        self.host, self.memo = HostOnly(), {}

    def infer_type(self, base_type, transforms):
        key = (id(base_type), id(transforms))
        if key not in self.memo:
            self.memo[key] = (self.host.infer_type(base_type, transforms), base_type, transforms)
        return self.memo[key][0]


class NoTransport:
    def setup(self, sf):
        return 0


def _workloads():
    return {"llama7b": W.llama7b_decls(layers=4), "cfg1": W.conv_weight_decls(24), "cfg2": W.int4_linear_decls(3),
            "cfg3": W.sparse_conv_decls(12), "cfg4": W.resnet_decls(2)}


@pytest.fixture(scope="module")
def host():
    return CachedHost()


@pytest.fixture(scope="module")
def workloads():
    return _workloads()


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("name", ["llama7b", "cfg1", "cfg2", "cfg3", "cfg4"])
@pytest.mark.parametrize("shares", ["ingress-aware", "equal"])
def test_layout_tiles_the_blob(host, workloads, name, world, shares):
    decls = workloads[name]
    weights = None if shares == "ingress-aware" else [1.0] * world
    nchunks = 4 if shares == "ingress-aware" else 7
    rank0_chunks = 1 if shares == "ingress-aware" else 7
    folders = [ShardedFolder(host, decls, r, world, NoTransport(), weights=weights, nchunks=nchunks,
                             folder_cls=SlotsOnly, rank0_chunks=rank0_chunks) for r in range(world)]
    L = folders[0].layout
    n = len(decls)
    sizes = [host.infer_type(d.base_type, d.transforms).getTotalAllocSize() for d in decls]

    # one owner per constant, the chunks of a rank are its constants in model order
    assert sorted(i for r in range(world) for i in L.mine[r]) == list(range(n))
    for r in range(world):
        assert [i for c in L.chunks[r] for i in c] == L.mine[r]
        assert all(c for c in L.chunks[r]) and len(L.chunks[r]) <= (rank0_chunks if r == 0 else nchunks)
    assert L.nchunks == max(1, max(len(c) for c in L.chunks))

    # regions follow one another, chunks follow one another inside a region, all on slot boundaries
    at = 0
    for r in range(world):
        assert L.region_off[r] == at and at % SEGMENT_ALIGN == 0
        assert all(o % SEGMENT_ALIGN == 0 for o in L.chunk_off[r])
        assert L.chunk_off[r] == sorted(L.chunk_off[r]) and (not L.chunk_off[r] or L.chunk_off[r][0] == 0)
        at += L.region_bytes[r]
    assert L.blob_bytes == max(at, 1)

    # every slot of every rank: inside its chunk's span, disjoint from every other slot
    spans = []
    for r, sf in enumerate(folders):
        assert sf.layout.owner == L.owner and sf.layout.region_off == L.region_off and sf.layout.chunk_off == L.chunk_off
        assert sf.layout.table_row_of == L.table_row_of and sf.layout.flags_off == L.flags_off
        for k, chunk in enumerate(sf.my_chunks):
            lo, nbytes = sf.chunk_span(r, k)
            for i, off in zip(chunk, sf._slot_off[k]):
                assert lo <= off and off + sizes[i] <= lo + nbytes
                spans.append((off, off + sizes[i], i))
    spans.sort()
    assert [s[2] for s in sorted(spans, key=lambda s: s[2])] == list(range(n))
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
    assert spans[-1][1] <= L.blob_bytes

    # table rows: one per constant, grouped rank by rank in chunk order; table and sequence words behind the blob
    assert sorted(L.table_row_of.values()) == list(range(n))
    rows_in_order = [L.table_row_of[i] for r in range(world) for c in L.chunks[r] for i in c]
    assert rows_in_order == list(range(n))
    assert L.table_off >= L.blob_bytes and L.table_off % 256 == 0
    assert L.flags_off >= L.table_off + n * Layout.TABLE_ROW * 8 and L.flags_off % 256 == 0
    assert L.buffer_bytes == L.flags_off + L.nchunks * world * 8


@pytest.fixture(scope="module")
def full_model():
    return W.llama7b_decls(layers=32)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_shares_follow_the_weights(host, workloads, full_model, world):
    decls = full_model
    total = sum(d.nbytes for d in decls)
    for f in (0.5, 0.7, 0.9):
        weights = [f] + [(1.0 - f) / (world - 1)] * (world - 1)
        L = Layout(decls, world, weights, 4, lambda i: decls[i].nbytes // 2)
        got = [sum(decls[i].nbytes for i in L.mine[r]) / total for r in range(world)]
        # longest-processing-time assignment: off by at most the largest constant (lm_head, 2 % of the model)
        assert np.allclose(got, weights, atol=0.025), (world, f, got)
        assert all(L.mine[r] for r in range(world))
    # the default shares keep rank 0 at or above an equal split and give the other ranks equal parts
    sf = ShardedFolder(host, workloads["llama7b"], 0, world, NoTransport(), folder_cls=SlotsOnly)
    assert sf.weights[0] >= 1.0 / world and len(set(round(w, 12) for w in sf.weights[1:])) == 1
    assert abs(sum(sf.weights) - 1.0) < 1e-9
