"""The benchmark's own inputs and outputs, byte for byte.

1. b200c_synth_fill (device generator) against the oracle's independent restatement of the same
   specification: identical bytes for every distribution and element type, plus the statistics the
   configurations ask for (sigma, zero fraction, clip range).
2. b200c_digest64_batch against the oracle's digest.
3. Every benchmark workload at its smallest count but FULL-SIZE shapes: inputs generated on the device,
   folded and compressed through the same ShardedFolder path the benchmark times, and every slot, size and
   compressed flag compared with the oracle run on the same input bytes.
"""
import numpy as np
import pytest

from npu_plugin_b200 import _cabi as A
from npu_plugin_b200 import workloads as W
from npu_plugin_b200.sharded import ShardedFolder, SingleTransport, blob_digest, combine_digests

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,dist,p0,p1,count", [
    (A.F32, 0, 0.05, 0.0, 1_000_003), (A.F16, 0, 0.02, 0.0, 2_000_001), (A.F16, 0, 1.0, 0.0, 4096),
    (A.SI8, 1, 0.5, 0.0, 1_048_576), (A.SI8, 1, 0.0, 0.0, 77), (A.SI8, 2, 12.0, 0.1, 3_000_002), (A.SI8, 2, 3.0, 0.3, 5),
])
def test_synth_fill_is_the_oracle_generator(gpu, oracle, dtype, dist, p0, p1, count):
    nbytes = count * A.dtype_bits(dtype) // 8
    dev = gpu.dev_alloc(nbytes)
    try:
        for seed, stream in ((5, 0), (5, 123456789012), (0xDEADBEEFCAFE, 7)):
            gpu.synth_fill(dev, count, dtype, dist, p0, p1, seed, stream)
            gpu.synchronize()
            got = gpu.download(dev, nbytes)
            want = oracle.synth_fill(count, dtype, dist, p0, p1, seed, stream)
            assert np.array_equal(got, want), f"generator bytes differ (seed {seed}, stream {stream})"
    finally:
        gpu.dev_free(dev)
    if count < 100_000:
        return
    # the distributions the configurations name
    if dist == 0:
        x = want.view(np.float32 if dtype == A.F32 else np.float16).astype(np.float64)
        assert abs(x.std() / p0 - 1.0) < 0.01 and abs(x.mean()) < 0.01 * p0
        assert abs(((x / p0) ** 4).mean() - 3.0) < 0.1          # normal kurtosis
        assert abs((np.abs(x) < p0).mean() - 0.6827) < 0.005
    elif dist == 1:
        x = want.view(np.int8)
        assert x.min() == -127 and x.max() == 127
        assert abs((x == 0).mean() - (p0 + (1 - p0) / 255)) < 0.005
    else:
        x = want.view(np.int8).astype(np.float64)
        assert x.min() >= -127 and x.max() <= 127
        natural_zero = 1.0 - np.exp(-0.5 / p0)
        assert abs((x == 0).mean() - (p1 + (1 - p1) * natural_zero)) < 0.01
        assert abs(np.abs(x[x != 0]).mean() / p0 - 1.0) < 0.1


def test_digest_is_the_oracle_digest(gpu, oracle):
    rng = np.random.default_rng(3)
    sizes = [0, 1, 7, 8, 9, 4096, 65536, 65537, 1_000_003, 8 * 8192 * 3]
    total = sum(sizes) + 64
    host = rng.integers(0, 256, total, dtype=np.uint8)
    dev = gpu.dev_alloc(total)
    try:
        gpu.upload(dev, host)
        for shift in (0, 1, 3):  # aligned and unaligned starts
            ptrs, at = [], shift
            for n in sizes:
                ptrs.append(dev + at)
                at += n
            got = gpu.digest64(ptrs, sizes)
            at = shift
            for n, g in zip(sizes, got):
                assert g == oracle.digest64(host[at:at + n]), f"digest of {n} bytes at offset {at}"
                at += n
    finally:
        gpu.dev_free(dev)


def test_detect_splat(gpu):
    rng = np.random.default_rng(4)
    for elem, n in ((1, 1_000_000), (2, 300_001), (4, 4099), (8, 70_000)):
        one = rng.integers(1, 255, elem, dtype=np.uint8)
        x = np.tile(one, n)
        assert gpu.detect_splat(x, elem)
        for where in (elem, (n // 2) * elem + elem - 1, n * elem - 1):
            y = x.copy()
            y[where] ^= 0x40
            assert not gpu.detect_splat(y, elem), f"elem {elem}: a difference at byte {where} went unnoticed"
        assert gpu.detect_splat(x[:elem], elem)          # a single element is a splat
    assert not gpu.detect_splat(np.zeros(0, np.uint8), 4)  # empty data is not
    from npu_plugin_b200.const import ConstError
    with pytest.raises(ConstError):
        gpu.detect_splat(np.zeros(6, np.uint8), 4)         # unexpected length
    with pytest.raises(ConstError):
        gpu.detect_splat(np.zeros(2, np.uint8), 4)         # less than one element


def _workload(name):
    if name == "llama1":
        return W.llama7b_decls(layers=1)
    return W.WORKLOADS[name][0](1)


@pytest.mark.parametrize("name", ["cfg1", "cfg2", "cfg3", "cfg4", "llama1"])
def test_benchmark_workload_at_full_size_shapes(gpu, oracle, name):
    decls = _workload(name)
    sf = ShardedFolder(gpu, decls, 0, 1, SingleTransport())
    owner, owners = W.shared_inputs(decls)  # the two constants of a sparse weight read one buffer
    own = {i: gpu.dev_alloc(decls[i].nbytes) for i in owners}
    ins = [own[o] for o in owner]
    side_bufs = []
    side = []
    for d in decls:
        if W.has_quantizer(d):
            s, z = gpu.dev_alloc(4 * d.base_type.shape[0]), gpu.dev_alloc(4 * d.base_type.shape[0])
            side_bufs += [s, z]
            side.append((s, z))
        else:
            side.append(None)
    try:
        for i in owners:
            W.fill_device(gpu, decls[i], own[i])
        gpu.synchronize()
        table = None
        for _ in range(2):  # twice: the second step overwrites streams left by the first
            rows = sf.step(ins, side, True)
            table = sf.collect(rows)
            sf.release()
        blob = gpu.download(sf.t.blob_ptr(), sf.layout.blob_bytes)
        assert [r[0] for r in table] == list(range(len(decls)))
        ref_digests, ref_table, compressed = [], [], 0
        slot_sizes = sf.folders[0].folded_sizes
        for k, ((i, off, size, comp), d, p) in enumerate(zip(table, decls, ins)):
            assert i == k
            x = oracle.synth_of(d, W.SEED)
            assert np.array_equal(gpu.download(p, d.nbytes), x), f"{d.name}: device input differs from the oracle generator"
            for t in d.transforms:
                if t.kind == A.X_QUANTIZE_SYNTH:
                    oc = d.base_type.shape[0]
                    t.side0, t.side1 = np.zeros(oc, np.float32), np.zeros(oc, np.int32)
            folded = oracle.fold(d.base_type, x, False, d.transforms).copyTo()
            # the slot as the reference's writer would leave it: a pre-zeroed buffer of the type's size with the
            # content copied in (a Sparsify<false> result is shorter than its type says)
            slot = np.zeros(slot_sizes[k], np.uint8)
            slot[:folded.size] = folded
            live, ref_comp = slot, False
            if d.compress and slot.size >= 4096:
                stream, not_smaller = oracle.btc_compress(slot)
                if not not_smaller:
                    live, ref_comp = stream, True
            compressed += ref_comp
            assert (size, bool(comp)) == (live.size, ref_comp), f"{d.name}: size / compressed flag differ from the oracle"
            assert np.array_equal(blob[off:off + size], live), f"{d.name}: blob bytes differ from the oracle"
            for t in d.transforms:
                if t.kind == A.X_QUANTIZE_SYNTH:  # the per-channel scale table is part of the output
                    assert np.array_equal(gpu.download(side[k][0], 4 * d.base_type.shape[0]).view(np.float32), t.side0)
                    t.side0 = t.side1 = None
            ref_table.append((i, off, live.size, ref_comp))
            ref_digests.append(oracle.digest64(live))
        if name == "cfg4":
            assert compressed >= 40, "the Laplace-distributed ResNet weights should compress"
        # the digest the benchmark prints is the one the oracle's bytes give
        assert blob_digest(gpu, sf.t.blob_ptr(), table) == combine_digests(ref_digests, ref_table)
    finally:
        for p in list(own.values()) + side_bufs:
            gpu.dev_free(p)
        sf.close()
