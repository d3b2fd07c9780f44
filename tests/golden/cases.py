"""Seeded small instances of the five benchmark configurations and of the codec, shared by the fixture
generator (make_fixtures.py) and the fixture test (tests/test_golden_fixtures.py)."""
import numpy as np

from npu_plugin_b200 import _cabi as A
from npu_plugin_b200.const import ContentAttr, DimsOrder, NDType, UniformQuantizedPerAxisType


def _q8(o, expressed):
    return UniformQuantizedPerAxisType(A.SI8, expressed, [1.0] * o, [0] * o, 0, -127, 127)


def conv_weight(backend, seed=1, shape=(32, 48, 3, 3)):
    w = np.random.default_rng(seed).normal(0, 0.05, shape).astype(np.float32)
    a = ContentAttr.get(w, NDType(shape, A.F32), backend=backend).quantizeSynth(A.QSYNTH_SYM_I8)
    a = a.convertElemType(A.SI8).quantCast(_q8(shape[0], A.F32)).reorder(DimsOrder.OYXI)
    return a.padWithZero((0, 0, 0, 0), (0, (-shape[1]) % 16, 0, 0)).swizzleConstant(5, 3)


def int4_linear(backend, seed=2, shape=(96, 512)):
    w = np.random.default_rng(seed).normal(0, 0.02, shape).astype(np.float16)
    o = shape[0]
    a = ContentAttr.get(w, NDType(shape + (1, 1), A.F16), backend=backend).quantizeSynth(A.QSYNTH_ASYM_U4)
    q = UniformQuantizedPerAxisType(A.UI8, A.F16, [1.0] * o, [0] * o, 0, 0, 15)
    return a.convertElemType(A.UI8).quantCast(q).reorder(DimsOrder.NHWC).bitPack(4)


def dequantize(backend, seed=3, shape=(40, 256)):
    rng = np.random.default_rng(seed)
    x = rng.integers(0, 16, shape).astype(np.uint8)
    o = shape[0]
    q = UniformQuantizedPerAxisType(A.UI8, A.F16, list(rng.uniform(0.001, 0.01, o)), [int(v) for v in rng.integers(0, 16, o)],
                                    0, 0, 15)
    return ContentAttr.get(x, NDType(shape, A.UI8), backend=backend).quantCast(q).dequantize()


def _sparse_weights(seed, shape):
    rng = np.random.default_rng(seed)
    x = rng.integers(-127, 128, shape).astype(np.int8)
    x[rng.random(shape) < 0.5] = 0
    return x


def sparsity_map(backend, seed=4, shape=(64, 128, 1, 1)):
    x = _sparse_weights(seed, shape)
    return ContentAttr.get(x, NDType(shape, A.SI8), backend=backend).getSparsityMap().swizzleConstant(5, 3)


def sparsify(backend, seed=4, shape=(64, 128, 1, 1)):
    x = _sparse_weights(seed, shape)
    return ContentAttr.get(x, NDType(shape, A.SI8), backend=backend).sparsify(False).swizzleConstant(5, 3)


def resnet_weight(backend, seed=5, shape=(64, 64, 3, 3)):
    rng = np.random.default_rng(seed)
    x = np.clip(np.rint(rng.laplace(0, 12.0, shape)), -127, 127).astype(np.int8)
    x[rng.random(shape) < 0.1] = 0
    a = ContentAttr.get(x, NDType(shape, A.SI8), backend=backend).quantCast(_q8(shape[0], A.F16))
    return a.reorder(DimsOrder.OYXI)


def llama_linear(backend, seed=6, shape=(48, 1024)):
    w = np.random.default_rng(seed).normal(0, 0.02, shape).astype(np.float16)
    a = ContentAttr.get(w, NDType(shape + (1, 1), A.F16), backend=backend).quantizeSynth(A.QSYNTH_SYM_I8)
    a = a.convertElemType(A.SI8).quantCast(_q8(shape[0], A.F16)).reorder(DimsOrder.NHWC)
    return a.swizzleConstant(5, 3)


CASES = {
    "cfg1_conv_weight": (conv_weight, False),
    "cfg2_int4_pack": (int4_linear, False),
    "cfg2_dequantize": (dequantize, False),
    "cfg3_sparsity_map": (sparsity_map, False),
    "cfg3_sparsify": (sparsify, False),
    "cfg4_resnet_weight_compressed": (resnet_weight, True),
    "cfg5_llama_linear_compressed": (llama_linear, True),
}


def run_case(name, backend):
    """Folds the case on `backend`; returns the folded bytes and, for compressed cases, the stream
    (or None when the codec reports that the stream is not smaller)."""
    build, compress = CASES[name]
    folded = np.ascontiguousarray(build(backend).fold().copyTo()).view(np.uint8).ravel()
    stream = None
    if compress:
        out, not_smaller = backend.btc_compress(folded)
        stream = None if not_smaller else np.asarray(out, np.uint8)
    return folded, stream
