#!/usr/bin/env python
"""Benchmark of the weight-preparation hot path on B200.

Workload (default): whole-model fold of a 7B Llama-shaped decoder with synthetic f16 weights: every
linear weight goes through per-output-channel symmetric int8 quantisation -> ConvertElemType ->
QuantCast -> Reorder -> SwizzleConstant(5) and then block compression; embedding and RMSNorm gains
pass through.  Constants are sharded by tensor over the ranks; finished slots are pushed into one
blob on rank 0 over NVLink.  A "step" is one pass over the whole model.

  python bench.py --gpus N --steps K --warmup W            # this library (N>1 under torchrun)
  python bench.py --impl reference ...                      # the CPU path (oracle) on the host cores

Prints ONE JSON line (rank 0).
"""
import argparse
import ctypes as C
import datetime
import gc
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

from npu_plugin_b200 import _cabi as A  # noqa: E402
from npu_plugin_b200 import workloads as W  # noqa: E402
from npu_plugin_b200.sharded import PushTransport, ShardedFolder, SingleTransport, combine_digests  # noqa: E402

HBM_FALLBACK_GBS = 6650.0
# DRAM bytes per algorithmic byte of the dominant kernel, from one ncu capture per workload on a reduced
# case (traffic grows in proportion to the rows processed); None: no capture for that workload
DRAM_PER_ALGORITHMIC_BYTE = {"llama7b": (576.79 + 259.20) / (576.72 + 288.36 + 0.56)}


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms",
                                          "50", "-i", str(self.index)], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, reasons = [], set()
        try:
            for line in open(self.path):
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1]))
                    out["sm_max_mhz"] = float(p[2])
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out["sm_mhz"] = float(np.median(sm))
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return HBM_FALLBACK_GBS, "fallback"


# ----------------------------------------------------------------------------- CPU (reference arm / cpu_baseline)
def cpu_sample_decls(decls, budget_elems):
    """A bounded sample of the workload for the host: whole tensors, in model order, up to the element limit."""
    out, total = [], 0
    for i, d in enumerate(decls):
        if not d.transforms:
            continue
        n = d.base_type.getNumElements()
        if out and total + n > budget_elems:
            break
        out.append(i)
        total += n
    return out


def run_cpu(decls, steps, warmup, budget_elems, threads=None, want_digests=False):
    """Times the CPU restatement of the reference's folding + codec (oracle) on a bounded sample whose
    inputs are the same bytes the device generator produces.  Returns (GB/s over algorithmic bytes, ms per
    sample pass, cores, sample description, {constant index: (digest, size, compressed)})."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_backend import OracleBackend
    orc = OracleBackend()
    cores = orc.set_threads(threads or (os.cpu_count() or 1))
    sample = cpu_sample_decls(decls, budget_elems)
    data = [orc.synth_of(decls[i], W.SEED) for i in sample]
    slot_sizes = {i: orc.infer_type(decls[i].base_type, decls[i].transforms).getTotalAllocSize() for i in sample}
    for i in sample:
        for t in decls[i].transforms:
            if t.kind == A.X_QUANTIZE_SYNTH:
                oc = decls[i].base_type.shape[0]
                t.side0, t.side1 = np.zeros(oc, np.float32), np.zeros(oc, np.int32)
    times, bytes_step, digests = [], 0, {}
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        b = 0
        results = []
        for i, x in zip(sample, data):
            d = decls[i]
            folded = orc.fold(d.base_type, x, False, d.transforms).copyTo()
            b += d.nbytes + folded.size
            if W.has_quantizer(d):
                b += 4 * d.base_type.shape[0]
            # the constant's buffer as the reference's writers hold it: pre-zeroed, of the type's size, with the
            # content copied in (a Sparsify result is shorter than its type says)
            slot_size = slot_sizes[i]
            if folded.size < slot_size:
                slot = np.zeros(slot_size, np.uint8)
                slot[:folded.size] = folded
                folded = slot
            live, comp = folded, False
            if d.compress and folded.size >= 4096:
                stream, not_smaller = orc.btc_compress(folded)
                b += folded.size + (0 if not_smaller else stream.size)
                if not not_smaller:
                    live, comp = stream, True
            results.append((i, live, comp))
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
            bytes_step = b
        if want_digests and it == warmup + steps - 1:  # outside the timed passes' clocks
            digests = {i: (orc.digest64(live), int(live.size), bool(comp)) for i, live, comp in results}
    for i in sample:
        for t in decls[i].transforms:
            t.side0 = t.side1 = None
    sec = float(np.mean(times))
    desc = f"the first {len(sample)} constants of the workload ({sum(decls[i].base_type.getNumElements() for i in sample)} elements), fold + codec"
    return bytes_step / sec / 1e9, sec * 1e3, cores, desc, digests


# ----------------------------------------------------------------------------- one workload on the device
class DeviceRun:
    """Inputs resident in HBM, one ShardedFolder, CUDA-event timing of K steps."""

    def __init__(self, torch, dist, backend, stream, decls, rank, world, comm, args, rank0_chunks=1, weights=None):
        self.torch, self.dist, self.b, self.stream = torch, dist, backend, stream
        self.decls, self.rank, self.world = decls, rank, world
        transport = PushTransport(comm, timeout_ms=args.exchange_timeout_ms, mode=args.push_mode, ctas=args.push_ctas) \
            if world > 1 else SingleTransport()
        self.sf = ShardedFolder(backend, decls, rank, world, transport, weights=weights, nchunks=args.chunks,
                                rank0_chunks=rank0_chunks)
        self.mine = [decls[i] for i in self.sf.layout.mine[rank]]
        owner, owners = W.shared_inputs(self.mine)
        self.inputs = {i: torch.empty(self.mine[i].nbytes, dtype=torch.uint8, device="cuda") for i in owners}
        for i in owners:
            W.fill_device(backend, self.mine[i], self.inputs[i].data_ptr())
        self.in_ptrs = [self.inputs[o].data_ptr() for o in owner]
        hq = [W.has_quantizer(d) for d in self.mine]
        self.scales = [torch.empty(d.base_type.shape[0], dtype=torch.float32, device="cuda") if q else None
                       for d, q in zip(self.mine, hq)]
        self.zps = [torch.empty(d.base_type.shape[0], dtype=torch.int32, device="cuda") if q else None
                    for d, q in zip(self.mine, hq)]
        self.side = [(s.data_ptr(), z.data_ptr()) if s is not None else None for s, z in zip(self.scales, self.zps)]
        self.table = None
        self.issue_s = 0.0

    def step(self, timers=None):
        """One pass; timers = (begin, end, {(name, chunk): event})."""
        stream = self.stream
        if timers:
            timers[0].record(stream)
        t0 = [0.0]

        def hooks(name, k):
            if name == "fold0":
                t0[0] = time.perf_counter()
            elif name == "fold1":
                self.issue_s += time.perf_counter() - t0[0]
            if timers:
                ev = self.torch.cuda.Event(enable_timing=True)
                ev.record(stream)
                timers[2][(name, k)] = ev

        rows = self.sf.step(self.in_ptrs, self.side, True, hooks)
        if self.rank == 0:
            self.table = self.sf.collect(rows)  # bounded waits on the stream, then the table
            if timers:
                timers[1].record(stream)
            self.sf.release()
        else:
            self.own_rows = rows
            if timers:
                timers[1].record(stream)

    def sync_all(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def timed(self, steps, warmup):
        torch = self.torch
        for _ in range(max(warmup, 0)):
            self.step()
        self.sync_all()
        launches0 = self.b.launch_count()

        def mk():
            return torch.cuda.Event(enable_timing=True)

        ev = [(mk(), mk(), {}) for _ in range(steps)]
        t_begin, t_end = mk(), mk()
        self.issue_s = 0.0
        t_begin.record(self.stream)
        for k in range(steps):
            self.step(ev[k])
        t_end.record(self.stream)
        self.sync_all()
        self.sf.t.check(self.sf)
        out = {"elapsed_ms": t_begin.elapsed_time(t_end), "launches": self.b.launch_count() - launches0,
               "issue_ms": self.issue_s * 1e3 / max(1, steps)}
        nchunks = len(self.sf.folders)
        out["fold_ms"] = float(np.mean([sum(e[2][("fold0", k)].elapsed_time(e[2][("fold1", k)]) for k in range(nchunks)) for e in ev]))
        out["codec_ms"] = float(np.mean([sum(e[2][("fold1", k)].elapsed_time(e[2][("codec1", k)]) for k in range(nchunks)) for e in ev]))
        out["step_ms_local"] = float(np.mean([e[0].elapsed_time(e[1]) for e in ev]))
        return out

    def byte_counts(self):
        """(fold bytes, codec bytes, compressed constants, blob bytes) of this rank's share."""
        own = {i: (size, comp) for i, _, size, comp in (self.table if self.rank == 0 else self.own_rows)}
        idx = self.sf.layout.mine[self.rank]
        # bytes the fold really wrote (a Sparsify result is shorter than its slot) and the slot sizes the codec reads
        written = [f for fl in self.sf.folders for f in fl.written_sizes()]
        slots = [f for fl in self.sf.folders for f in fl.folded_sizes]
        streams = [own[i][0] if own[i][1] else None for i in idx]
        fold_b, codec_b = W.algorithmic_bytes(self.mine, written, streams, slots)
        return fold_b, codec_b, sum(1 for i in idx if own[i][1]), sum(own[i][0] for i in idx), written

    def fold_launches(self):
        l0 = self.b.launch_count()
        at = 0
        for k, (chunk, f) in enumerate(zip(self.sf.my_chunks, self.sf.folders)):
            n = len(chunk)
            f.fold(self.in_ptrs[at:at + n], self.sf.local_base + self.sf.layout.chunk_off[self.rank][k], True, self.side[at:at + n])
            at += n
        self.torch.cuda.synchronize()
        return int(self.b.launch_count() - l0)

    def kernels_only_ms(self, steps=5):
        """Device time of the fold phase when the host has a head start (a spin kernel occupies the stream
        while the launches are queued), plus the codec phase as timed by events."""
        torch = self.torch
        tot = 0.0
        for _ in range(steps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(int(8e6))  # a few ms at ~2 GHz
            a.record(self.stream)
            at = 0
            for k, (chunk, f) in enumerate(zip(self.sf.my_chunks, self.sf.folders)):
                n = len(chunk)
                f.fold(self.in_ptrs[at:at + n], self.sf.local_base + self.sf.layout.chunk_off[self.rank][k], True, self.side[at:at + n])
                at += n
            b.record(self.stream)
            torch.cuda.synchronize()
            tot += a.elapsed_time(b)
        return tot / steps

    def close(self):
        self.sf.close()
        del self.inputs, self.scales, self.zps


class Comm:
    """Host-side set-up exchange of the transport (object all-gather on a gloo group)."""

    def __init__(self, dist, group, world):
        self.dist, self.group, self.world = dist, group, world

    def all_gather(self, obj):
        out = [None] * self.world
        self.dist.all_gather_object(out, obj, group=self.group)
        return out


def run_e2e(torch, dist, backend, stream, decls, rank, world, comm, args, algorithmic_bytes, weights):
    """The same metric through the C ABI with host buffers.  Every step: host -> device copy of this rank's
    inputs from pinned memory (inside b200c_fold_batch), fold, compress, push to rank 0, and on rank 0 the
    device -> host copy of the whole blob into pinned memory (b200c_copy_segments_async)."""
    # For the end-to-end job the PCIe links are the bound: every rank uploads over its own link, so the
    # inputs are split evenly unless a share was asked for.
    w = weights if weights is not None else ([1.0] * world)
    transport = PushTransport(comm, timeout_ms=args.exchange_timeout_ms, mode=args.push_mode, ctas=args.push_ctas) \
        if world > 1 else SingleTransport()
    total_in = sum(d.nbytes for d in decls)
    chunk_bytes = args.e2e_chunk_bytes
    nchunks = max(1, min(16, (total_in // world + chunk_bytes - 1) // chunk_bytes))
    sf = ShardedFolder(backend, decls, rank, world, transport, weights=w, nchunks=nchunks, rank0_chunks=nchunks)
    mine = [decls[i] for i in sf.layout.mine[rank]]
    owner, owners = W.shared_inputs(mine)
    host_own = {i: torch.empty(mine[i].nbytes, dtype=torch.uint8, pin_memory=True) for i in owners}
    tmp = torch.empty(max([d.nbytes for d in mine] + [1]), dtype=torch.uint8, device="cuda")
    for i in owners:
        W.fill_device(backend, mine[i], tmp.data_ptr())
        host_own[i].copy_(tmp[:mine[i].nbytes])
    host_in = [host_own[o] for o in owner]
    torch.cuda.synchronize()
    del tmp
    hq = [W.has_quantizer(d) for d in mine]
    scales = [torch.empty(d.base_type.shape[0], dtype=torch.float32, device="cuda") if q else None for d, q in zip(mine, hq)]
    zps = [torch.empty(d.base_type.shape[0], dtype=torch.int32, device="cuda") if q else None for d, q in zip(mine, hq)]
    side = [(a.data_ptr(), z.data_ptr()) if a is not None else None for a, z in zip(scales, zps)]
    host_blob = torch.empty(sf.layout.blob_bytes, dtype=torch.uint8, pin_memory=True) if rank == 0 else None
    in_ptrs = [h.data_ptr() for h in host_in]
    state = {"d2h": 0, "table": None}

    def step():
        d2h = [0]

        def hooks(name, k):
            # rank 0's chunk k is complete: it goes home, and so do the peers' chunks k once they have arrived,
            # while the next chunk uploads
            if name == "codec1" and rank == 0:
                d2h[0] += sf.download_chunk(host_blob.data_ptr(), k)

        rows = sf.step(in_ptrs, side, False, hooks, max_batch_bytes=1 << 30)
        if rank == 0:
            d2h[0] += sf.download(host_blob.data_ptr(), first_chunk=len(sf.folders))
            state["table"] = sf.collect(rows)
            backend.stream_join()  # the release follows the download of the blob
            sf.release()
            state["d2h"] = d2h[0]

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    step()
    sync_all()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(max(1, args.e2e_steps)):
        step()
    backend.stream_join()
    b.record(stream)
    sync_all()
    sf.t.check(sf)
    ems = a.elapsed_time(b) / max(1, args.e2e_steps)
    host_digest = None
    if world > 1:
        t = torch.tensor([ems], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ems = float(t.item())
    xfer = torch.tensor([sum(d.nbytes for d in mine), state["d2h"]], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(xfer)
    if rank == 0:
        # the blob that arrived in host memory, digested per constant like the device blob: one string at every N
        scratch = torch.empty(max(size for _, _, size, _ in state["table"]), dtype=torch.uint8, device="cuda")
        dg = []
        for _, off, size, _ in state["table"]:
            scratch[:size].copy_(host_blob[off:off + size])
            torch.cuda.synchronize()
            dg += backend.digest64([scratch.data_ptr()], [size])
        host_digest = combine_digests(dg, state["table"])
    out = {"value": algorithmic_bytes / (ems * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ems,
           "h2d_bytes_per_step": int(xfer[0].item()), "d2h_bytes_per_step": int(xfer[1].item()),
           "chunks": sf.layout.nchunks, "blob_digest_host": host_digest,
           "what": "host inputs -> b200c_fold_batch (upload inside) -> compress -> push to rank 0 -> download of the one blob"}
    sf.close()
    return out


def run_per_config(torch, dist, backend, stream, args, peak):
    """The four single-tensor configurations, batched (many independent instances per step), 20 timed steps
    each: value, time per step, the dominant kernel's phase fraction of the HBM roof and the fraction with
    the host's launch work taken out (fold kernels behind a head start + codec phase)."""
    out = {}
    for name in ("cfg1", "cfg2", "cfg3", "cfg4"):
        builder, n_inst, text, dtype_name, dominant = W.WORKLOADS[name]
        decls = builder(n_inst)
        run = DeviceRun(torch, dist, backend, stream, decls, 0, 1, None, args, rank0_chunks=W.PIPELINE_CHUNKS.get(name, 1))
        tm = run.timed(20, 3)
        fold_b, codec_b, n_comp, blob_b, folded_sizes = run.byte_counts()
        ms = tm["elapsed_ms"] / 20
        value = (fold_b + codec_b) / (ms * 1e-3) / 1e9
        ko_ms = run.kernels_only_ms() + tm["codec_ms"]
        phase_b, phase_ms = (codec_b, tm["codec_ms"]) if name == "cfg4" else (fold_b, tm["fold_ms"])
        out[name] = {"value": value, "unit": "GB/s", "ms_per_step": ms, "instances": n_inst, "dtype": dtype_name,
                     "frac": value / peak, "kernels_only_frac": (fold_b + codec_b) / (ko_ms * 1e-3) / 1e9 / peak,
                     "roofline": {"kernel": dominant, "frac": phase_b / (phase_ms * 1e-3) / 1e9 / peak if phase_ms > 0 else None,
                                  "phase": "codec" if name == "cfg4" else "fold"},
                     "phase_ms": {"fold": tm["fold_ms"], "codec": tm["codec_ms"], "fold_host_issue": tm["issue_ms"]},
                     "compressed_tensors": n_comp, "blob_bytes": blob_b}
        run.close()
        del run, decls
        torch.cuda.empty_cache()
    return out


# ----------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=32, help="decoder layers of the 7B-shape workload (32 = the named config)")
    ap.add_argument("--workload", default="llama7b", choices=["llama7b", "cfg1", "cfg2", "cfg3", "cfg4"],
                    help="llama7b = the whole-model configuration (the default bench line); cfgK = the K-th single-tensor "
                         "configuration, batched")
    ap.add_argument("--instances", type=int, default=None, help="independent instances per step for cfg1..cfg4")
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--e2e-chunk-bytes", type=int, default=1_500_000_000,
                    help="input bytes per chunk of the end-to-end leg (uploads, folds and downloads overlap chunk by chunk)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-per-config", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--cpu-sample-elements", type=int, default=220_000_000, help="elements of the CPU sample")
    ap.add_argument("--rank0-share", type=float, default=None,
                    help="share of the constants rank 0 keeps when several ranks push into its blob (default: balances its "
                         "compute against its NVLink ingress)")
    ap.add_argument("--chunks", type=int, default=4, help="chunks a pushing rank cuts its share into")
    ap.add_argument("--rank0-chunks", type=int, default=None,
                    help="chunks rank 0 cuts its share into (default: per workload; more than one lets the device "
                         "compress a chunk while the host plans the next)")
    ap.add_argument("--push-mode", type=int, default=2, choices=[0, 1, 2], help="0: copy kernel, 1: copy engine, 2: bulk-copy kernel")
    ap.add_argument("--push-ctas", type=int, default=32)
    ap.add_argument("--exchange-timeout-ms", type=int, default=20000)
    ap.add_argument("--log-tensors", default=None, help="write one JSON line per constant of the final blob to this file")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload == "llama7b":
        decls = W.llama7b_decls(layers=args.layers)
        workload = f"llama7b-shape fold: {len([d for d in decls if d.transforms])} linear f16 weights -> sym int8 per-channel " \
                   f"-> Reorder -> Swizzle(5) -> block codec; {len(decls)} constants, layers={args.layers}"
        config = {"workload": workload, "sharding": "by tensor (LPT; rank 0's share balances its compute against its ingress)",
                  "gather": "push over NVLink (owner's copy kernel into rank 0's blob)" if world > 1 else "none",
                  "l2": "per-step working set (>26 GB at N=1) exceeds L2", "layers": args.layers}
        dtype_name, dominant = "f16->i8", "rowQuantRegBatchKernel (fused quantise + reorder + swizzle, all tensors of a configuration per launch)"
    else:
        builder, default_n, text, dtype_name, dominant = W.WORKLOADS[args.workload]
        n_inst = args.instances or default_n
        decls = builder(n_inst)
        config = {"workload": f"{args.workload}: {text}; {n_inst} independent instances per step",
                  "sharding": "by tensor (LPT)", "l2": "instances rotate through buffers larger than L2", "instances": n_inst}

    if args.impl == "reference":
        if rank != 0:
            return
        gbs, ms, cores, desc, _ = run_cpu(decls, max(1, args.steps), max(0, args.warmup), args.cpu_sample_elements)
        line = {"impl": "reference", "metric": "folded_weight_GBps", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": dtype_name, "data": "synthetic", "config": config,
                "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": desc},
                "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    import torch
    import torch.distributed as dist
    from npu_plugin_b200.const import CudaBackend

    torch.cuda.set_device(local_rank)
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        # host-side group: only the set-up exchange of the IPC descriptors goes through it; a short time limit
        # turns a stuck set-up into an error instead of a hang
        pg_host = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=180))
        comm = Comm(dist, pg_host, world)
    # the planning threads of all ranks share the host's cores
    os.environ.setdefault("B200C_PLAN_THREADS", str(max(1, min(8, (os.cpu_count() or 8) // (2 * world)))))
    backend = CudaBackend(local_rank)
    lib, ctx = backend.lib, backend.ctx
    # a real (non-default) stream shared by torch and the library, so that torch's CUDA events are
    # recorded on the stream the kernels are launched on
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    assert stream.cuda_stream != 0
    lib.b200c_set_stream(ctx, C.c_void_p(stream.cuda_stream))

    weights = None
    if args.rank0_share is not None and world > 1:
        f = min(0.98, max(1.0 / world, args.rank0_share))
        weights = [f] + [(1.0 - f) / (world - 1)] * (world - 1)

    # The workload description holds millions of Python objects (per-channel scale lists); a cyclic
    # garbage collection walking them would stall the host in the middle of a step.
    # rank 0 cuts its share into chunks only where the compression of one chunk can hide the host's planning of
    # the next (workloads of many small constants); its slots never travel
    run = DeviceRun(torch, dist, backend, stream, decls, rank, world, comm, args, weights=weights,
                    rank0_chunks=args.rank0_chunks or W.PIPELINE_CHUNKS.get(args.workload, 1))
    gc.collect()
    gc.freeze()
    sampler = ClockSampler(local_rank)
    sampler.start()  # sampled from the warm-up on: the timed region can be shorter than nvidia-smi's start-up
    tm = run.timed(args.steps, args.warmup)
    clocks = sampler.stop()
    elapsed_ms, launches = tm["elapsed_ms"], tm["launches"]
    if world > 1:
        t = torch.tensor([elapsed_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
        ln = torch.tensor([launches], dtype=torch.int64, device="cuda")
        dist.all_reduce(ln)
        launches = int(ln.item())
    ms_per_step = elapsed_ms / args.steps
    fold_ms, codec_ms = tm["fold_ms"], tm["codec_ms"]
    gather_ms = max(0.0, tm["step_ms_local"] - fold_ms - codec_ms)  # exposed (not hidden) part of the exchange
    per_rank = None
    if world > 1:  # every rank's own view of the timed region: [ms per step, fold, codec] on its stream
        mine_t = torch.tensor([tm["elapsed_ms"] / args.steps, fold_ms, codec_ms], dtype=torch.float64, device="cuda")
        all_t = [torch.zeros_like(mine_t) for _ in range(world)]
        dist.all_gather(all_t, mine_t)
        per_rank = [[round(float(x), 3) for x in t.tolist()] for t in all_t]

    # algorithmic bytes of the whole job (all ranks)
    fold_b, codec_b, n_comp, blob_local, folded_sizes = run.byte_counts()
    tot = torch.tensor([fold_b, codec_b, n_comp, blob_local], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(tot)
    fold_all, codec_all, n_compressed, blob_bytes = [float(x) for x in tot.tolist()]
    value = (fold_all + codec_all) / (ms_per_step * 1e-3) / 1e9

    # the assembled blob, digested per constant (outside the timed region): the same string at every N
    digest, gpu_results = None, {}
    if rank == 0:
        blob = run.sf.t.blob_ptr()
        gpu_digests = backend.digest64([blob + off for _, off, _, _ in run.table], [size for _, _, size, _ in run.table])
        digest = combine_digests(gpu_digests, run.table)
        gpu_results = {i: (dg, size, bool(comp)) for dg, (i, _, size, comp) in zip(gpu_digests, run.table)}
        if args.log_tensors:
            from npu_plugin_b200.sharded import tensor_log_lines
            sizes = {}
            for r in range(world):
                for chunk in run.sf.layout.chunks[r]:
                    for i in chunk:
                        sizes[i] = backend.infer_type(decls[i].base_type, decls[i].transforms).getTotalAllocSize()
            with open(args.log_tensors, "w") as f:
                f.write("\n".join(tensor_log_lines(decls, run.table, sizes.get)) + "\n")

    # roofline of the dominant kernel
    peak, peak_kind = measured_peak()
    n_fold_launch = run.fold_launches()
    fold_local_b, _ = W.algorithmic_bytes(run.mine, folded_sizes, [None] * len(run.mine))
    achieved = fold_local_b / (fold_ms * 1e-3) / 1e9 if fold_ms > 0 else 0.0
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None, "peak_kind": peak_kind, "kernel": dominant,
                "launches_per_step": n_fold_launch, "avg_launch_ms": fold_ms / max(1, n_fold_launch),
                "tensors_per_step": len([d for d in run.mine if d.transforms]),
                "algorithmic_bytes_per_launch": fold_local_b / max(1, n_fold_launch),
                "phase_ms": {"fold": fold_ms, "codec": codec_ms, "gather": gather_ms, "fold_host_issue": tm["issue_ms"]},
                "per_rank_ms": per_rank}
    ratio = DRAM_PER_ALGORITHMIC_BYTE.get(args.workload)
    if ratio is not None:
        roofline["traffic"] = ratio * roofline["algorithmic_bytes_per_launch"]
        roofline["traffic_source"] = "ncu capture of a smaller case of this workload, scaled by algorithmic bytes"
    layout_info = {"rank0_share": run.sf.weights[0] if world > 1 else 1.0, "chunks": run.sf.layout.nchunks,
                   "constants_per_rank": [len(m) for m in run.sf.layout.mine]}
    run.close()
    del run
    torch.cuda.empty_cache()

    # end to end through the C ABI with host buffers (pinned): every rank uploads its own share over its own
    # PCIe link, folds, compresses and pushes; rank 0 downloads the assembled blob into host memory, chunk by
    # chunk as the chunks complete.  Both copies are inside the timed region.
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(torch, dist, backend, stream, decls, rank, world, comm, args, fold_all + codec_all, weights)

    per_config = None
    if rank == 0 and world == 1 and args.workload == "llama7b" and not args.no_per_config:
        per_config = run_per_config(torch, dist, backend, stream, args, peak)

    cpu, verified = None, None
    if rank == 0 and world == 1 and not args.no_cpu:
        # one untimed pass first: page faults, thread start-up
        gbs, ms, cores, desc, cpu_digests = run_cpu(decls, 1, 1, args.cpu_sample_elements, want_digests=True)
        cpu = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": desc, "ms_per_sample": ms}
        # the checker: the blob bytes the timed steps produced for the sampled constants equal the oracle's
        ok = bool(cpu_digests) and all(cpu_digests[i] == gpu_results.get(i) for i in cpu_digests)
        verified = {"constants": len(cpu_digests), "match": bool(ok), "against": "CPU oracle on the same generated bytes"}

    if rank == 0:
        line = {"metric": "folded_weight_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": dtype_name, "data": "synthetic", "config": config, "clocks": clocks,
                "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline, "cpu_baseline": cpu,
                "bytes": {"fold": fold_all, "codec": codec_all, "blob": blob_bytes, "compressed_tensors": n_compressed},
                "per_gpu_GBps": value / world, "blob_digest": digest, "verified": verified, "layout": layout_info,
                "per_config": per_config}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
