"""CPU-side checks of the C ABI: the library loads, exports every symbol include/b200const.h declares,
and its host-only entry points (type inference, insertion order, sizes) agree with the oracle.  No
compute entry point is called here."""
import os
import re

import numpy as np
import pytest

from npu_plugin_b200 import _cabi as A
from npu_plugin_b200 import const as K
from npu_plugin_b200.const import DimsOrder, NDType, Transform, UniformQuantizedPerAxisType, UniformQuantizedType

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class HostOnly:
    """The library's host entry points behind the backend interface (no context, no device)."""

    def __init__(self):
        self.lib = A.load()

    def infer_type(self, base_type, transforms):
        return K.infer_type_through(self.lib.b200c_infer_type, self.lib.b200c_last_error, base_type, transforms)

    def insert_position(self, kinds, new_kind):
        import ctypes as C
        arr = (C.c_int32 * max(1, len(kinds)))(*kinds)
        pos = C.c_int()
        K.raise_for(self.lib.b200c_insert_position(arr, len(kinds), new_kind, C.byref(pos)), self.lib.b200c_last_error())
        return pos.value


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "b200const.h")).read()
    declared = set(re.findall(r"B200C_API\s+[\w\s\*]+?\b(b200c_\w+)\s*\(", header))
    assert len(declared) >= 25
    assert declared == set(A.SYMBOLS), declared ^ set(A.SYMBOLS)
    lib = A.load()
    for name in declared:
        assert hasattr(lib, name), name
    assert b"sm_100a" in lib.b200c_version()


def test_create_fails_loudly_without_a_device():
    import ctypes as C
    try:
        import torch
        if torch.cuda.is_available():
            pytest.skip("a GPU is present")
    except ImportError:
        pass
    lib = A.load()
    h = C.c_void_p()
    assert lib.b200c_create(0, C.byref(h)) == A.ERR_CUDA
    assert b"CUDA" in lib.b200c_last_error() or b"device" in lib.b200c_last_error()


CHAINS = [
    ((4, 6, 3, 3), A.F32, DimsOrder.NCHW, [Transform(A.X_CONVERT_ELEM_TYPE, elem=A.SI8), Transform(A.X_REORDER, a=DimsOrder.NHWC),
                                           Transform(A.X_PAD_WITH_ZERO, a=(0, 0, 0, 0), b=(0, 10, 0, 0)),
                                           Transform(A.X_SWIZZLE_CONSTANT, i0=5, i1=3)]),
    ((8, 16, 1, 1), A.UI8, DimsOrder.NCHW, [Transform(A.X_QUANT_CAST, elem=UniformQuantizedPerAxisType(A.UI8, A.F16, [0.5] * 8, [3] * 8, 0)),
                                            Transform(A.X_PAD_WITH_ZERO, a=(1, 0, 0, 0), b=(2, 0, 0, 0)),
                                            Transform(A.X_SUBVIEW, a=(1, 0, 0, 0), b=(4, 16, 1, 1)), Transform(A.X_DEQUANTIZE)]),
    ((2, 8, 2, 2), A.SI8, DimsOrder.NHWC, [Transform(A.X_QUANT_CAST, elem=UniformQuantizedType(A.SI8, A.F32, 0.1, 0)),
                                           Transform(A.X_GET_SPARSITY_MAP), Transform(A.X_SWIZZLE_CONSTANT, i0=5, i1=3)]),
    ((2, 8, 2, 2), A.F16, DimsOrder.NCHW, [Transform(A.X_SPARSIFY, i0=1, aux=[5, 17])]),
    ((6, 4), A.F16, DimsOrder.NC, [Transform(A.X_TRANSPOSE, a=(1, 0)), Transform(A.X_RESHAPE, b=(1, 4, 6, 1)),
                                   Transform(A.X_BIT_PACK, i0=4)]),
    ((1, 9, 2), A.F32, DimsOrder.CHW, [Transform(A.X_RESHAPE, b=(1, 3, 3, 2)), Transform(A.X_BROADCAST, i0=0, i1=4)]),
    ((4, 3, 5, 5), A.SI8, DimsOrder.NCHW, [Transform(A.X_QUANT_CAST, elem=UniformQuantizedType(A.SI8, A.F16, 0.25, 3)),
                                           Transform(A.X_EXPAND_DILATED, a=(2, 3)), Transform(A.X_REVERSE, i0=1)]),
    ((16, 1, 1, 4), A.SI32, DimsOrder.NCHW, [Transform(A.X_RELOCATE_WEIGHTS_TABLE, a=(0, 8), b=(100, 200), i0=5000)]),
]


@pytest.mark.parametrize("case", range(len(CHAINS)))
def test_type_inference_matches_oracle(oracle, case):
    shape, dt, order, chain = CHAINS[case]
    base = NDType(shape, dt, order)
    host = HostOnly()
    for k in range(len(chain) + 1):
        try:
            exp = oracle.infer_type(base, chain[:k])
        except K.ConstError:
            with pytest.raises(K.ConstError):
                host.infer_type(base, chain[:k])
            continue
        assert host.infer_type(base, chain[:k]) == exp


def test_insert_position_matches_oracle(oracle):
    host = HostOnly()
    kinds_pool = [A.X_RESCALE, A.X_REORDER, A.X_SPARSIFY, A.X_GET_SPARSITY_MAP, A.X_BIT_PACK, A.X_SWIZZLE_CONSTANT]
    rng = np.random.default_rng(0)
    for _ in range(200):
        kinds = []
        for _ in range(int(rng.integers(0, 6))):
            new = int(rng.choice(kinds_pool))
            try:
                pe = oracle.insert_position(kinds, new)
            except K.ConstError:
                with pytest.raises(K.ConstError):
                    host.insert_position(kinds, new)
                continue
            assert host.insert_position(kinds, new) == pe
            kinds.insert(pe, new)


def test_errors_of_type_inference(oracle):
    host = HostOnly()
    base = NDType((2, 4), A.F32)
    for backend in (host, oracle):
        with pytest.raises(K.ConstError):
            backend.infer_type(base, [Transform(A.X_DEQUANTIZE)])
        with pytest.raises(K.ConstError):
            backend.infer_type(base, [Transform(A.X_BIT_PACK, i0=4)])
        with pytest.raises(K.ConstError):
            backend.infer_type(base, [Transform(A.X_GET_SPARSITY_MAP)])
        with pytest.raises(K.ConstError):
            backend.infer_type(base, [Transform(A.X_QUANT_CAST, elem=UniformQuantizedType(A.UI8, A.F32, 1.0, 0))])


def test_type_inference_asks_again_when_the_parameter_storage_is_short(oracle, monkeypatch):
    """The library reports how many quantisation parameters the output type holds; the host layer's second call
    brings exactly that storage, so a low first guess costs one more call and changes nothing in the result."""
    host = HostOnly()
    oc = 300
    q = UniformQuantizedPerAxisType(A.SI8, A.F16, [0.5 + 0.001 * k for k in range(oc)], [3] * oc, 0, -128, 127)
    base = NDType((oc, 16, 1, 1), A.SI8)
    chain = [Transform(A.X_QUANT_CAST, elem=q), Transform(A.X_PAD_WITH_ZERO, a=(0, 0, 0, 0), b=(7, 0, 0, 0)),
             Transform(A.X_REORDER, a=DimsOrder.NHWC)]
    want = oracle.infer_type(base, chain)
    assert len(want.quant.scales) == oc + 7
    assert host.infer_type(base, chain) == want
    calls = []
    monkeypatch.setattr(K, "quick_q_of", lambda b, t: calls.append(1) or 1)
    assert host.infer_type(base, chain) == want and calls
    assert oracle.infer_type(base, chain) == want  # the oracle's binding asks again the same way
    # an unquantised result needs no storage at all
    assert host.infer_type(base, chain + [Transform(A.X_DEQUANTIZE)]) == oracle.infer_type(base, chain + [Transform(A.X_DEQUANTIZE)])
