"""Constant fusion and the constants-section writers.

The oracle (oracle/fusion_oracle.py) is pinned by the fused sizes, element types and hex bytes the reference's
lit test holds (tests/golden/fuse_constants_vectors.json, extracted from
tests/lit/NPU/dialect/VPUIP/passes/fuse_constants.mlir); the GPU path (npu_plugin_b200.fusion) is compared with the
same vectors and with the oracle."""
import json
import os
import sys

import numpy as np
import pytest

from npu_plugin_b200 import _cabi as A
from npu_plugin_b200.const import ContentAttr, DimsOrder, NDType, UniformQuantizedType

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import fusion_oracle  # noqa: E402

CASES = json.load(open(os.path.join(ROOT, "tests", "golden", "fuse_constants_vectors.json")))["cases"]
ELEM = {"si32": (A.SI32, np.int32), "f16": (A.F16, np.float16), "ui8": (A.UI8, np.uint8)}


def build_attr(entry, case, backend):
    """ContentAttr of one constant of a lit case."""
    shape = tuple(entry["shape"])
    dt, npdt = ELEM[entry["elem"]]
    if "hex" in entry:
        arr = np.frombuffer(bytes.fromhex(entry["hex"]), np.uint8).view(npdt).reshape(shape)
        a = ContentAttr.get(arr, NDType(shape, dt), backend=backend)
    elif "values" in entry:
        a = ContentAttr.get(np.array(entry["values"], npdt).reshape(shape), NDType(shape, dt), backend=backend)
    else:
        a = ContentAttr.get(np.array([entry["splat"]], npdt), NDType(shape, dt), is_splat=True, backend=backend)
    for t in entry["transforms"]:
        if t == "#const.Reorder<#NHWC>":
            a = a.reorder(DimsOrder.NHWC)
        elif t == "#const.Sparsify<false>":
            a = a.sparsify(False)
        elif t == "#const.GetSparsityMap":
            a = a.getSparsityMap()
        elif t == "#const.ConvertElemType<si8>":
            a = a.convertElemType(A.SI8)
        elif t == "#const.QuantCast<!qElemType>":
            q = case["qElemType"]
            a = a.quantCast(UniformQuantizedType(A.SI8, A.F16, q["scale"], 0, q["qmin"], q["qmax"]))
        else:
            raise AssertionError(t)
    return a


def kind_of(t):
    from npu_plugin_b200.fusion import _part_kind
    return _part_kind(t)


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_reproduces_the_pinned_fused_constants(oracle, case):
    parts = []
    for key in ("weight_table", "weights", "weights_sm", "activation_window"):
        e = case["constants"].get(key)
        if e is None:
            parts.append(None)
            continue
        a = build_attr(e, case, oracle)
        parts.append((a.fold().copyTo(), kind_of(a.getType())))
    fused, elem, n, views = fusion_oracle.fuse_constants(parts)
    assert (elem, n) == (case["fused_elem_type"], case["fused_elems"])
    if case["fused_hex"]:
        assert fused.tobytes().hex().upper() == case["fused_hex"].upper()
    at = 0
    for v in views:
        if v is not None:
            assert v[0] == at
            at += v[1]
    assert at == n


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_gpu_fusion_matches_the_pinned_vectors_and_the_oracle(gpu, oracle, case):
    from npu_plugin_b200.fusion import fuse_constants
    attrs, parts = {}, []
    for key in ("weight_table", "weights", "weights_sm", "activation_window"):
        e = case["constants"].get(key)
        attrs[key] = build_attr(e, case, gpu) if e else None
        if e:
            o = build_attr(e, case, oracle)
            parts.append((o.fold().copyTo(), kind_of(o.getType())))
        else:
            parts.append(None)
    got = fuse_constants(gpu, **attrs)
    want, elem, n, views = fusion_oracle.fuse_constants(parts)
    assert got.type.shape == (1, 1, 1, case["fused_elems"])
    assert got.type.dtype == (A.F16 if case["fused_elem_type"] == "f16" else A.UI8)
    assert np.array_equal(got.data, want)
    assert got.views == views
    if case["fused_hex"]:
        assert got.data.tobytes().hex().upper() == case["fused_hex"].upper()


def test_section_writers_oracle():
    rng = np.random.default_rng(1)
    consts = [rng.integers(0, 256, n, dtype=np.uint8) for n in (5, 8, 13, 4096, 1)]
    data, offs = fusion_oracle.graph_schema_section(consts)
    assert offs == [0, 8, 16, 32, 4128] and data.size == 4136
    for c, o in zip(consts, offs):
        assert np.array_equal(data[o:o + c.size], c)
        assert not data[o + c.size:(o + c.size + 7) // 8 * 8].any()
    data, offs = fusion_oracle.elf_section(consts)
    assert offs == [0, 5, 13, 26, 4122] and data.size == 4123


@pytest.mark.gpu
@pytest.mark.parametrize("align", [8, 1])
def test_gpu_section_writer(gpu, align):
    from npu_plugin_b200.fusion import write_section
    rng = np.random.default_rng(2)
    sizes = [5, 8, 13, 4096, 1, 70_001, 512]
    blob_host = rng.integers(0, 256, 512 * 400, dtype=np.uint8)
    table, at = [], 0
    for i, s in enumerate(sizes):
        table.append((i, at, s, i % 2))
        at = (at + s + 511) // 512 * 512
    blob = gpu.dev_alloc(blob_host.size)
    try:
        gpu.upload(blob, blob_host)
        sec = write_section(gpu, blob, table, align=align)
    finally:
        gpu.dev_free(blob)
    consts = [blob_host[o:o + s] for _, o, s, _ in table]
    want, offs = (fusion_oracle.graph_schema_section if align == 8 else fusion_oracle.elf_section)(consts)
    assert sec.offsets == offs and np.array_equal(sec.data, want)
