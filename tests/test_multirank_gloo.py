"""The multi-rank path on CPU: two gloo ranks shard a list of constants with the library's partition rule
and gather their blob segments on rank 0 with the same exchange routine bench.py uses over NCCL."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, tmpdir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from npu_plugin_b200 import _cabi as A
    from npu_plugin_b200.blob import ConstantDecl, gather_segments, partition
    from npu_plugin_b200.const import NDType

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sizes = [4096 * 4096, 11008 * 4096, 4096 * 11008, 32000 * 4096, 4096, 4096 * 4096, 11008 * 4096]
        decls = [ConstantDecl(f"c{i}", NDType((n,), A.F16), [], 2 * n) for i, n in enumerate(sizes)]
        owner = partition(decls, world)
        mine = [i for i, o in enumerate(owner) if o == rank]
        # each rank's "blob": its constants' ids repeated, so the assembled order can be checked
        parts = [np.full(16 + 7 * i, i, np.uint8) for i in mine]
        local = np.concatenate(parts) if parts else np.zeros(0, np.uint8)
        blob = torch.zeros(local.size + 100, dtype=torch.uint8)
        blob[:local.size] = torch.from_numpy(local)
        for _ in range(2):  # twice: the receive buffer is reused
            szs, gathered = gather_segments(dist, blob, local.size, rank, world)
        np.save(os.path.join(tmpdir, f"owner{rank}.npy"), np.array(owner))
        if rank == 0:
            np.save(os.path.join(tmpdir, "gathered.npy"), gathered[:sum(szs)].numpy())
            np.save(os.path.join(tmpdir, "sizes.npy"), np.array(szs))
        else:
            assert gathered is None
    finally:
        dist.destroy_process_group()


def test_two_rank_shard_and_gather(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    o0, o1 = np.load(tmp_path / "owner0.npy"), np.load(tmp_path / "owner1.npy")
    assert np.array_equal(o0, o1), "ranks disagree on the partition"
    assert set(o0.tolist()) == {0, 1}
    got = np.load(tmp_path / "gathered.npy")
    sizes = np.load(tmp_path / "sizes.npy")
    expect = np.concatenate([np.full(16 + 7 * i, i, np.uint8) for r in range(2) for i in range(len(o0)) if o0[i] == r])
    assert sizes.sum() == expect.size
    assert np.array_equal(got, expect)
