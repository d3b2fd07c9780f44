"""The folding cache and background folding (npu_plugin_b200.cache), shaped like the reference's unit test
tests/unit/vpux_compiler/dialect/const/constant_folding_in_background_tests.cpp:62-130: 1 to 5 folding threads,
one compilation and two concurrent compilations under different contexts, results equal to a direct fold.  Plus
what the device-resident cache adds: partial folds that start from the cached prefix, and the cases in which a
prefix must NOT be reused (pending lazy conversion, splat)."""
import threading
import time

import numpy as np
import pytest

from npu_plugin_b200 import _cabi as A
from npu_plugin_b200.cache import (ConstantFoldingCacheManager, initBackgroundConstantFoldingThreads, prefix_is_reusable,
                                   stopBackgroundConstantFoldingThreads)
from npu_plugin_b200.const import ContentAttr, DimsOrder, NDType


def same_transformation(backend):
    base = np.full(100, 1.0, np.float32)
    a = ContentAttr.get(base, backend=backend)
    for _ in range(5):
        a = a.add(1.0)
    return a, np.full(100, 6.0, np.float32)


def mixed_transformations(backend):
    base = np.zeros(100, np.float32)
    a = ContentAttr.get(base, backend=backend).padWithZero((10,), (10,)).add(1.0).rescale(3.0).subview((0,), (100,))
    return a, np.full(100, 3.0, np.float32)


def compile_under(ctx, num_threads, sleep_s, make):
    threads = initBackgroundConstantFoldingThreads(ctx, num_threads, collectStatistics=True)
    attr, expected = make(ctx)
    time.sleep(sleep_s)
    got = attr.fold().copyTo().view(np.float32)
    stats = stopBackgroundConstantFoldingThreads(ctx, threads, collectStatistics=True)
    assert np.array_equal(got, expected)
    assert np.array_equal(attr.fold(bypassCache=True).copyTo().view(np.float32), expected)
    return stats


def new_context(backend):
    """A second compilation context on the same kind of backend."""
    if backend.name == "oracle":
        from oracle_backend import OracleBackend
        return OracleBackend()
    from npu_plugin_b200.const import CudaBackend
    return CudaBackend(backend.device)


@pytest.mark.parametrize("num_threads", [1, 2, 3, 4, 5])
def test_compilation_flow(backend, num_threads):
    ctx = new_context(backend)
    stats = compile_under(ctx, num_threads, 0.1, same_transformation)
    assert stats["cache hits"] >= 1
    assert not ConstantFoldingCacheManager.getInstance().contains(ctx)


@pytest.mark.parametrize("num_threads", [1, 3, 5])
def test_multiple_compilations(backend, num_threads):
    ctxs = [new_context(backend), new_context(backend)]
    errors = []

    def run(ctx, sleep_s, make):
        try:
            compile_under(ctx, num_threads, sleep_s, make)
        except Exception as e:  # pragma: no cover
            errors.append(e)

    ts = [threading.Thread(target=run, args=(ctxs[0], 0.1, same_transformation)),
          threading.Thread(target=run, args=(ctxs[1], 0.3, mixed_transformations))]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert not errors, errors


def test_partial_folds_reuse_the_cached_prefix(backend):
    ctx = new_context(backend)
    threads = initBackgroundConstantFoldingThreads(ctx, 1, collectStatistics=True)
    rng = np.random.default_rng(5)
    w = rng.normal(0, 1, (8, 16, 3, 3)).astype(np.float32)
    a = ContentAttr.get(w, backend=ctx)
    chain = a.add(0.5).rescale(2.0).reorder(DimsOrder.NHWC).padWithZero((0, 0, 0, 0), (0, 16, 0, 0))
    got = chain.fold().copyTo()
    stats = stopBackgroundConstantFoldingThreads(ctx, threads, collectStatistics=True)
    assert np.array_equal(got, chain.fold(bypassCache=True).copyTo())
    # every step after the first was folded on top of its predecessor's cached content, which was then dropped
    assert stats["partial folds"] == 3
    assert stats["elements erased"] == 3


def test_prefix_with_pending_conversion_or_splat_is_not_reused(backend):
    ctx = new_context(backend)
    w = np.array([0.1, 1.0 / 3.0, 2.5, 1000.123], np.float32)
    a = ContentAttr.get(w, backend=ctx)
    lazy = a.convertElemType(A.F16)           # storage f32, logical f16: conversion still pending
    assert not prefix_is_reusable(lazy)
    assert prefix_is_reusable(a.add(1.0))     # storage f32, logical f32
    assert not prefix_is_reusable(lazy.rescale(3.0))  # rescale allocates f32 storage; the logical type stays f16
    splat = ContentAttr.get(np.array([2.0], np.float32), NDType((4, 4), A.F32), is_splat=True, backend=ctx)
    assert not prefix_is_reusable(splat.add(1.0))
    threads = initBackgroundConstantFoldingThreads(ctx, 2, collectStatistics=True)
    # rescale sees the ORIGINAL f32 values (one rounding to f16 at the end), not the f16-rounded prefix
    chain = ContentAttr.get(w, backend=ctx).convertElemType(A.F16).rescale(3.0)
    got = chain.fold().copyTo().view(np.float16)
    stats = stopBackgroundConstantFoldingThreads(ctx, threads, collectStatistics=True)
    want = (w * np.float32(3.0)).astype(np.float16)
    assert np.array_equal(got, want)
    assert np.array_equal(got, chain.fold(bypassCache=True).copyTo().view(np.float16))
    assert stats["partial folds"] == 0


def test_failing_request_raises_in_the_foreground(backend):
    from npu_plugin_b200.const import ConstError
    ctx = new_context(backend)
    threads = initBackgroundConstantFoldingThreads(ctx, 1)
    bad = ContentAttr.get(np.array([300.0, 1.0], np.float32), backend=ctx).convertElemType(A.UI8)  # 300 does not fit
    with pytest.raises(ConstError):
        bad.fold()
    stopBackgroundConstantFoldingThreads(ctx, threads)
