#!/usr/bin/env python
"""Benchmark of the weight-preparation hot path on B200.

Workload (default): whole-model fold of a 7B Llama-shaped decoder with synthetic f16 weights
(BASELINE.json configs[4]): every linear weight goes through per-output-channel symmetric int8
quantisation -> ConvertElemType -> QuantCast -> Reorder -> SwizzleConstant(5) and then block
compression; embedding and RMSNorm gains pass through.  Constants are sharded by tensor over the
ranks; compressed segments are gathered on rank 0.  A "step" is one pass over the whole model.

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
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

from npu_plugin_b200 import _cabi as A  # noqa: E402
from npu_plugin_b200.blob import ConstantDecl, PeerWindow, ShardFolder, gather_aware_weights, partition  # noqa: E402
from npu_plugin_b200.const import (DimsOrder, NDType, Transform, UniformQuantizedPerAxisType,  # noqa: E402
                                   UniformQuantizedType)

DRAM_PER_ALGORITHMIC_BYTE = (576.79 + 259.20) / (576.72 + 288.36 + 0.56)
HBM_FALLBACK_GBS = 6650.0


# ----------------------------------------------------------------------------- workload
def llama7b_decls(layers=32, hidden=4096, ffn=11008, vocab=32000):
    """225 linear weights + embedding + 65 RMSNorm gains of a 7B Llama-shaped decoder (shapes only)."""
    decls = []

    def linear(name, o, i):
        q = UniformQuantizedPerAxisType(A.SI8, A.F16, [1.0] * o, [0] * o, 0, -127, 127)
        chain = [Transform(A.X_QUANTIZE_SYNTH, i0=A.QSYNTH_SYM_I8), Transform(A.X_CONVERT_ELEM_TYPE, elem=A.SI8),
                 Transform(A.X_QUANT_CAST, elem=q), Transform(A.X_REORDER, a=DimsOrder.NHWC),
                 Transform(A.X_SWIZZLE_CONSTANT, i0=5, i1=3)]
        decls.append(ConstantDecl(name, NDType((o, i, 1, 1), A.F16), chain, o * i * 2, compress=True))

    for l in range(layers):
        for n in ("q", "k", "v", "o"):
            linear(f"l{l}.{n}", hidden, hidden)
        linear(f"l{l}.gate", ffn, hidden)
        linear(f"l{l}.up", ffn, hidden)
        linear(f"l{l}.down", hidden, ffn)
    linear("lm_head", vocab, hidden)
    decls.append(ConstantDecl("embedding", NDType((vocab, hidden), A.F16), [], vocab * hidden * 2, compress=False))
    for l in range(2 * layers + 1):
        decls.append(ConstantDecl(f"norm{l}", NDType((hidden,), A.F16), [], hidden * 2, compress=False))
    return decls


def conv_weight_decls(instances):
    """configs[0]: f32 [256,256,3,3] -> sym int8 per-channel -> OIYX->OYXI -> pad I to x16 -> Swizzle(5)."""
    decls = []
    for k in range(instances):
        q = UniformQuantizedPerAxisType(A.SI8, A.F32, [1.0] * 256, [0] * 256, 0, -127, 127)
        chain = [Transform(A.X_QUANTIZE_SYNTH, i0=A.QSYNTH_SYM_I8), Transform(A.X_CONVERT_ELEM_TYPE, elem=A.SI8),
                 Transform(A.X_QUANT_CAST, elem=q), Transform(A.X_REORDER, a=DimsOrder.OYXI),
                 Transform(A.X_PAD_WITH_ZERO, a=(0, 0, 0, 0), b=(0, 0, 0, 0)), Transform(A.X_SWIZZLE_CONSTANT, i0=5, i1=3)]
        d = ConstantDecl(f"conv{k}", NDType((256, 256, 3, 3), A.F32), chain, 256 * 256 * 9 * 4, compress=False)
        d.synth = (A.F32, 0, 0.05, 0.0)
        decls.append(d)
    return decls


def int4_linear_decls(instances):
    """configs[1]: f16 [11008,4096] -> asym u4 per-channel -> BitPack (-> NHWC); and a Dequantize leg
    u8 [11008,4096] -> per-axis QuantCast -> Dequantize -> f16."""
    decls = []
    O, I = 11008, 4096
    for k in range(instances):
        q = UniformQuantizedPerAxisType(A.UI8, A.F16, [1.0] * O, [0] * O, 0, 0, 15)
        chain = [Transform(A.X_QUANTIZE_SYNTH, i0=A.QSYNTH_ASYM_U4), Transform(A.X_CONVERT_ELEM_TYPE, elem=A.UI8),
                 Transform(A.X_QUANT_CAST, elem=q), Transform(A.X_REORDER, a=DimsOrder.NHWC), Transform(A.X_BIT_PACK, i0=4)]
        d = ConstantDecl(f"pack{k}", NDType((O, I, 1, 1), A.F16), chain, O * I * 2, compress=False)
        d.synth = (A.F16, 0, 0.02, 0.0)
        decls.append(d)
        qd = UniformQuantizedPerAxisType(A.UI8, A.F16, [0.001 + 1e-6 * (j % 97) for j in range(O)], [j % 16 for j in range(O)], 0, 0, 15)
        chain = [Transform(A.X_QUANT_CAST, elem=qd), Transform(A.X_REORDER, a=DimsOrder.NHWC), Transform(A.X_DEQUANTIZE)]
        d = ConstantDecl(f"dequant{k}", NDType((O, I, 1, 1), A.UI8), chain, O * I, compress=False)
        d.synth = (A.SI8, 1, 0.0, 0.0)
        decls.append(d)
    return decls


def sparse_conv_decls(instances):
    """configs[2]: int8 [1024,1024,1,1], 50 % zeros -> GetSparsityMap -> Swizzle and Sparsify -> Swizzle."""
    decls = []
    for k in range(instances):
        for name, chain in (("map", [Transform(A.X_GET_SPARSITY_MAP), Transform(A.X_SWIZZLE_CONSTANT, i0=5, i1=3)]),
                            ("vals", [Transform(A.X_SPARSIFY, i0=0), Transform(A.X_SWIZZLE_CONSTANT, i0=5, i1=3)])):
            d = ConstantDecl(f"{name}{k}", NDType((1024, 1024, 1, 1), A.SI8), chain, 1024 * 1024, compress=False)
            d.synth = (A.SI8, 1, 0.5, 0.0)
            d.stream = k  # both chains of an instance see the same weights
            decls.append(d)
    return decls


def resnet50_shapes():
    shapes = [(64, 3, 7, 7)]
    inplanes = 64
    for width, blocks in ((64, 3), (128, 4), (256, 6), (512, 3)):
        for b in range(blocks):
            shapes += [(width, inplanes, 1, 1), (width, width, 3, 3), (width * 4, width, 1, 1)]
            if b == 0:
                shapes.append((width * 4, inplanes, 1, 1))
            inplanes = width * 4
    shapes.append((1000, 2048, 1, 1))
    return shapes


def resnet_decls(instances):
    """configs[3]: 53 conv + fc int8 weights -> QuantCast -> OIYX->OYXI (-> pad I to x16) -> block codec."""
    decls = []
    for k in range(instances):
        for j, (o, i, y, x) in enumerate(resnet50_shapes()):
            q = UniformQuantizedType(A.SI8, A.F16, 0.01, 0, -127, 127)
            chain = [Transform(A.X_QUANT_CAST, elem=q), Transform(A.X_REORDER, a=DimsOrder.OYXI)]
            if i % 16 and i < 16:
                chain.append(Transform(A.X_PAD_WITH_ZERO, a=(0, 0, 0, 0), b=(0, 16 - i % 16, 0, 0)))
            d = ConstantDecl(f"r{k}.{j}", NDType((o, i, y, x), A.SI8), chain, o * i * y * x, compress=True)
            d.synth = (A.SI8, 2, 12.0, 0.1)
            decls.append(d)
    return decls


def algorithmic_bytes(decls, folded_sizes, stream_sizes):
    """Read-once + write-once bytes of one step.  Fold: input + folded output (written straight into
    the blob slot) + scale tables.  Codec: every constant offered to it is read once; only a stream
    that is smaller than its constant is written (stream_sizes[i] is its length, else None)."""
    fold = sum(d.nbytes for d in decls) + sum(folded_sizes)
    fold += sum(4 * d.base_type.shape[0] for d in decls if any(t.kind == A.X_QUANTIZE_SYNTH for t in d.transforms))
    codec = 0
    for d, fs, ss in zip(decls, folded_sizes, stream_sizes):
        if d.compress and fs >= 4096:
            codec += fs + (ss or 0)
    return fold, codec


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
def host_data(d, rng):
    """Host copy of a constant's synthetic values (same distributions as the device generator)."""
    dt, kind, p0, p1 = getattr(d, "synth", (A.F16, 0, 0.02, 0.0))
    n = d.base_type.getNumElements()
    if kind == 0:
        return rng.normal(0, p0, n).astype(np.float32 if dt == A.F32 else np.float16)
    if kind == 1:
        x = rng.integers(-127, 128, n).astype(np.int8)
        x[rng.random(n) < p0] = 0
        return x
    x = np.clip(np.rint(rng.laplace(0, p0, n)), -127, 127).astype(np.int8)
    x[rng.random(n) < p1] = 0
    return x


def cpu_sample_decls(decls, budget_elems):
    """A bounded sample of the workload for the host: whole tensors, in model order, up to the element limit."""
    out, total = [], 0
    for d in decls:
        if not d.transforms:
            continue
        n = d.base_type.getNumElements()
        if out and total + n > budget_elems:
            break
        out.append(d)
        total += n
    return out


def run_cpu(decls, steps, warmup, budget_elems, threads=None):
    """Times the CPU restatement of the reference's folding + codec (oracle) on a bounded sample.
    Returns (GB/s over algorithmic bytes, ms per sample pass, cores, sample description)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_backend import OracleBackend
    orc = OracleBackend()
    cores = orc.set_threads(threads or (os.cpu_count() or 1))
    sample = cpu_sample_decls(decls, budget_elems)
    rng = np.random.default_rng(5)
    data = [host_data(d, rng) for d in sample]
    side = [(np.zeros(d.base_type.shape[0], np.float32), np.zeros(d.base_type.shape[0], np.int32)) for d in sample]
    for d, s in zip(sample, side):
        for t in d.transforms:
            if t.kind == A.X_QUANTIZE_SYNTH:
                t.side0, t.side1 = s
    times, bytes_step = [], 0
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        b = 0
        for d, x in zip(sample, data):
            c = orc.fold(d.base_type, x, False, d.transforms)
            folded = c.copyTo()
            b += d.nbytes + folded.size
            if any(t.kind == A.X_QUANTIZE_SYNTH for t in d.transforms):
                b += 4 * d.base_type.shape[0]
            if d.compress and folded.size >= 4096:
                stream, not_smaller = orc.btc_compress(folded)
                b += folded.size + (0 if not_smaller else stream.size)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
            bytes_step = b
    for d in sample:
        for t in d.transforms:
            t.side0 = t.side1 = None
    sec = float(np.mean(times))
    desc = f"the first {len(sample)} constants of the workload ({sum(d.base_type.getNumElements() for d in sample)} elements), fold + codec"
    return bytes_step / sec / 1e9, sec * 1e3, cores, desc


# ----------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=32, help="decoder layers of the 7B-shape workload (32 = the named config)")
    ap.add_argument("--workload", default="llama7b", choices=["llama7b", "cfg1", "cfg2", "cfg3", "cfg4"],
                    help="llama7b = BASELINE configs[4] (the default bench line); cfgK = configs[K-1], batched")
    ap.add_argument("--instances", type=int, default=None, help="independent instances per step for cfg1..cfg4")
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--gather", default="auto", choices=["auto", "pull", "nccl"],
                    help="multi-rank exchange: rank 0 pulls peers' slots through CUDA IPC with device copies, or NCCL "
                         "send/recv; auto = NCCL for two ranks (one peer: its copy kernels cost less than they gain), pull beyond")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--cpu-sample-elements", type=int, default=220_000_000, help="elements of the CPU sample")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gather == "auto":
        args.gather = "nccl" if world <= 2 else "pull"
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload == "llama7b":
        decls = llama7b_decls(layers=args.layers)
        workload = f"llama7b-shape fold: {len([d for d in decls if d.transforms])} linear f16 weights -> sym int8 per-channel " \
                   f"-> Reorder -> Swizzle(5) -> block codec; {len(decls)} constants, layers={args.layers}"
        config = {"workload": workload, "sharding": "by tensor (LPT; rank 0's share balances its compute against its ingress)", "gather": args.gather, "l2": "per-step working set (>26 GB at N=1) exceeds L2",
                  "layers": args.layers}
        dtype_name = "f16->i8"
    else:
        builder, default_n, text = {
            "cfg1": (conv_weight_decls, 512, "conv weight f32 [256,256,3,3] -> sym int8 -> OYXI -> pad -> Swizzle(5)"),
            "cfg2": (int4_linear_decls, 8, "f16 [11008,4096] -> asym u4 -> BitPack; and u8 -> per-axis Dequantize -> f16"),
            "cfg3": (sparse_conv_decls, 512, "int8 [1024,1024,1,1] 50% sparse -> sparsity map + sparsify, both Swizzle(5)"),
            "cfg4": (resnet_decls, 32, "ResNet-50-shaped int8 set (54 tensors) -> QuantCast -> OYXI (-> pad) -> block codec"),
        }[args.workload]
        n_inst = args.instances or default_n
        decls = builder(n_inst)
        config = {"workload": f"{args.workload}: {text}; {n_inst} independent instances per step",
                  "sharding": "by tensor (LPT)", "l2": "instances rotate through buffers larger than L2", "instances": n_inst}
        dtype_name = {"cfg1": "f32->i8", "cfg2": "f16->u4", "cfg3": "i8", "cfg4": "i8"}[args.workload]

    if args.impl == "reference":
        if rank != 0:
            return
        gbs, ms, cores, desc = run_cpu(decls, max(1, args.steps), max(0, args.warmup), args.cpu_sample_elements)
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
    if world > 1:
        # the segment transfers run on NCCL's own high-priority stream, so their kernels get SMs while
        # the fold kernels of the next chunk fill the machine
        # point-to-point transfers get the full set of channels whatever the number of ranks
        os.environ.setdefault("NCCL_MIN_P2P_NCHANNELS", "32")
        os.environ.setdefault("NCCL_MAX_P2P_NCHANNELS", "32")
        opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), pg_options=opts)
    # the planning threads of all ranks share the host's cores
    os.environ.setdefault("B200C_PLAN_THREADS", str(max(1, min(8, (os.cpu_count() or 8) // (2 * world)))))
    backend = CudaBackend(local_rank)
    lib, ctx = backend.lib, backend.ctx
    # a real (non-default) stream shared by torch and the library, so that torch's CUDA events are
    # recorded on the stream the kernels are launched on (the default stream's handle is 0, which
    # b200c_set_stream reads as "use the context's own stream")
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    assert stream.cuda_stream != 0
    lib.b200c_set_stream(ctx, C.c_void_p(stream.cuda_stream))

    # Every other rank's slots must enter rank 0 through its NVLink ingress, so rank 0 takes the larger
    # share of the constants: its compute time for that share balances the ingress time of the rest
    # (rates: 5 TB/s of algorithmic bytes for the kernels, 750 GB/s for the link; input bytes x 2 and x 0.5
    # approximate algorithmic and blob bytes of a constant before anything has run).  A larger share for
    # rank 0 measured worse: transfers crawl while rank 0's kernels keep its memory busy.
    total_in = sum(d.nbytes for d in decls)
    rate, link = 5.0e12, 0.75e12  # measured best at two ranks in both gather modes (rank 0 keeps 62.5 %)
    weights = gather_aware_weights(world, compute_seconds=2.0 * total_in / rate, transfer_seconds=0.5 * total_in / link)
    if args.gather == "pull" and world > 1:
        # copy-engine transfers into a GPU whose kernels saturate its memory make little progress until
        # those kernels end (measured), so compute and transfer add up instead of overlapping: rank 0 keeps
        # nearly everything and the peers take the rest
        weights = [0.9] + [0.1 / (world - 1)] * (world - 1)
    owner = partition(decls, world, weights)
    mine = [d for d, o in zip(decls, owner) if o == rank]
    folder = ShardFolder(backend, mine)  # whole-shard layout (sizes, bounds); also the N=1 path

    # device buffers (torch owns the memory; the library only sees pointers)
    inputs = [torch.empty(d.nbytes, dtype=torch.uint8, device="cuda") for d in mine]
    for i, d in enumerate(mine):
        dt, dist_kind, p0, p1 = getattr(d, "synth", (A.F16, 0, 0.02 if d.transforms else 1.0, 0.0))
        rc = lib.b200c_synth_fill(ctx, inputs[i].data_ptr(), d.nbytes * 8 // A.dtype_bits(dt), dt, dist_kind, p0, p1, 5,
                                  getattr(d, "stream", decls.index(d)))
        assert rc == 0, lib.b200c_last_error()
    in_ptrs = [t.data_ptr() for t in inputs]
    has_q = [any(t.kind == A.X_QUANTIZE_SYNTH for t in d.transforms) for d in mine]
    scales = [torch.empty(d.base_type.shape[0], dtype=torch.float32, device="cuda") if q else None for d, q in zip(mine, has_q)]
    zps = [torch.empty(d.base_type.shape[0], dtype=torch.int32, device="cuda") if q else None for d, q in zip(mine, has_q)]
    side = [(s.data_ptr(), z.data_ptr()) if s is not None else None for s, z in zip(scales, zps)]

    # With several ranks the shard is cut into chunks: while chunk c+1 is folded and compressed, chunk
    # c's segments already travel to rank 0 (NCCL send/recv over NVLink), so the gather hides behind
    # the compute as far as rank 0's ingress bandwidth allows.
    nchunks = 1 if world == 1 else (8 if args.gather == "pull" else 4)
    # rank 0's slots are produced where they stay, so in pull mode it has nothing to pipeline: one chunk
    my_chunks = 1 if (rank == 0 and args.gather == "pull") else nchunks
    per_chunk = (sum(d.nbytes for d in mine) + my_chunks - 1) // my_chunks if mine else 1
    chunks, cur, cur_bytes = [], [], 0
    for i, d in enumerate(mine):
        if cur and cur_bytes + d.nbytes > per_chunk and len(chunks) < my_chunks - 1:
            chunks.append(cur)
            cur, cur_bytes = [], 0
        cur.append(i)
        cur_bytes += d.nbytes
    chunks.append(cur)
    while len(chunks) < nchunks:
        chunks.append([])
    cf = [ShardFolder(backend, [mine[i] for i in c]) if c else None for c in chunks]
    fold_off, blob_off, fo, bo = [], [], 0, 0
    for f in cf:
        fold_off.append(fo)
        blob_off.append(bo)
        if f is not None:
            fo += f.folded_bytes
            bo += f.blob_bound
    # Every constant is folded straight into its slot of the blob; compression then works in place, so
    # the slot layout is known before any data is seen.  With several ranks the blob on rank 0 holds,
    # chunk after chunk, every rank's slots; rank 0 folds its own chunks directly into their final
    # place and receives the others' next to them.
    gathered, place = None, None
    if world > 1:
        # host-side group: chunk sizes at set-up, readiness notes and releases of the pull mode; a short
        # time limit turns a stuck exchange into an error instead of a hang
        pg_sizes = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=180))
        mine_sizes = torch.tensor([f.folded_bytes if f is not None else 0 for f in cf], dtype=torch.int64)
        all_sizes = [torch.zeros(nchunks, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(all_sizes, mine_sizes, group=pg_sizes)
        place, at = [[0] * world for _ in range(nchunks)], 0
        for k in range(nchunks):
            for r in range(world):
                place[k][r] = at
                at += int(all_sizes[r][k])
        # where chunk k starts inside rank r's own buffer (the running sum of its chunk sizes)
        peer_off = [[int(sum(int(all_sizes[r][j]) for j in range(k))) for k in range(nchunks)] for r in range(world)]
        if rank == 0:
            gathered = torch.empty(at + 1024, dtype=torch.uint8, device="cuda")
            folded = gathered
            fold_off = [place[k][0] for k in range(nchunks)]
        # the segment table (constant, offset, size, compressed) of every rank follows its last chunk
        counts = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(counts, torch.tensor([len(mine)], dtype=torch.int64), group=pg_sizes)
        tables = [torch.zeros((int(c.item()), 4), dtype=torch.int64, device="cuda") for c in counts] if rank == 0 else None
        my_table_host = torch.zeros((len(mine), 4), dtype=torch.int64, pin_memory=True)
        my_table = torch.zeros((len(mine), 4), dtype=torch.int64, device="cuda")
    if gathered is None:
        folded = torch.empty(max(fo, 1), dtype=torch.uint8, device="cuda")
    peers, copy_stream, gather_mode = None, None, "none"
    release = torch.zeros(1, dtype=torch.int64)
    if world > 1:
        # Pull mode: every peer exports its blob buffer; rank 0 maps them and copies ready chunks with
        # device-to-device copies on a stream of its own.  Readiness and release travel on the host (gloo).
        gather_mode = args.gather
        if gather_mode == "pull":
            ok = torch.ones(1, dtype=torch.int64)
            desc = None
            if rank:
                try:
                    desc = PeerWindow.export(folded)
                except Exception as e:
                    sys.stderr.write(f"[bench] rank {rank}: cannot export its buffer ({e})\n")
            descs = [None] * world
            dist.gather_object(desc, descs if rank == 0 else None, dst=0, group=pg_sizes)
            if rank == 0:
                try:
                    peers = [None] + [PeerWindow.open(d) for d in descs[1:]]
                    copy_stream = torch.cuda.Stream()
                    probe = torch.empty(16, dtype=torch.uint8, device="cuda")
                    for r in range(1, world):
                        probe.copy_(peers[r][:16])
                    torch.cuda.synchronize()
                except Exception as e:  # no peer mapping on this machine: NCCL send/recv instead
                    sys.stderr.write(f"[bench] peer windows unavailable ({e}); using NCCL send/recv\n")
                    ok[0] = 0
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=pg_sizes)
            if int(ok.item()) == 0:
                gather_mode, peers = "nccl", None
    seg_info = {}

    def step(timers=None):
        """One pass over the shard; timers = (begin, end, [per-chunk (fold0, fold1, codec1)]) CUDA events."""
        if timers:
            timers[0].record(stream)
        segs_all, used_total, pending, at = [], 0, [], 0
        puller = None
        if world > 1 and rank == 0:
            at = place[nchunks - 1][world - 1] + int(all_sizes[world - 1][nchunks - 1])
            if gather_mode == "pull":
                # a host thread waits for the peers' "chunk k is ready" notes (in the order they are sent)
                # and queues the copies on the copy stream while this thread folds rank 0's own chunks
                notes = [(k, r, torch.zeros(1, dtype=torch.int64)) for k in range(nchunks) for r in range(1, world)
                         if int(all_sizes[r][k])]
                reqs = [dist.irecv(t, src=r, group=pg_sizes) for k, r, t in notes]

                def pull():
                    torch.cuda.set_device(local_rank)
                    for (k, r, _), q in zip(notes, reqs):
                        q.wait()
                        n = int(all_sizes[r][k])
                        with torch.cuda.stream(copy_stream):
                            gathered[place[k][r]:place[k][r] + n].copy_(peers[r][peer_off[r][k]:peer_off[r][k] + n], non_blocking=True)

                copy_stream.wait_stream(stream)
                puller = threading.Thread(target=pull)
                puller.start()
            else:
                # every receive is posted before rank 0 starts its own work, chunk by chunk and peer by peer
                # (the order in which the peers send)
                for k in range(nchunks):
                    for r in range(1, world):
                        n = int(all_sizes[r][k])
                        if n:
                            pending.append(dist.irecv(gathered[place[k][r]:place[k][r] + n], src=r))
        for k, f in enumerate(cf):
            used = 0
            if f is not None:
                c = chunks[k]
                if timers:
                    timers[2][k][0].record(stream)
                h0 = time.perf_counter()
                f.fold([in_ptrs[i] for i in c], folded.data_ptr() + fold_off[k], True, [side[i] for i in c])
                seg_info["issue_s"] = seg_info.get("issue_s", 0.0) + (time.perf_counter() - h0)
                if timers:
                    timers[2][k][1].record(stream)
                segs = f.compress_inplace(folded.data_ptr() + fold_off[k])
                if timers:
                    timers[2][k][2].record(stream)
                used = f.folded_bytes  # the chunk's slots, streams and untouched constants alike
                segs_all += [(c[i], fold_off[k] + o, sz, comp) for i, o, sz, comp in segs]
            used_total += used
            if world > 1 and rank != 0 and used:
                if gather_mode == "pull":  # compress_inplace has synchronised: the chunk is complete
                    dist.send(torch.tensor([k], dtype=torch.int64), dst=0, group=pg_sizes)
                else:
                    pending.append(dist.isend(folded[fold_off[k]:fold_off[k] + used], dst=0))
        if world > 1 and gather_mode == "pull":
            # segment tables and the release of the peers' buffers travel on the host
            if rank == 0:
                puller.join()
                stream.wait_stream(copy_stream)
                if timers:
                    timers[1].record(stream)
                copy_stream.synchronize()
                tabs = [None] * world
                dist.gather_object(None, tabs, dst=0, group=pg_sizes)
                seg_info["tables"] = tabs
            else:
                if timers:
                    timers[1].record(stream)
                dist.gather_object(segs_all, None, dst=0, group=pg_sizes)
            # the peers may overwrite their buffers only after rank 0 has copied them
            dist.broadcast(release, src=0, group=pg_sizes)
            seg_info["segs"], seg_info["used"], seg_info["gathered"] = segs_all, used_total, at
            return
        if world > 1 and len(mine):
            if rank == 0:
                pending += [dist.irecv(tables[r], src=r) for r in range(1, world) if tables[r].numel()]
            else:
                my_table_host.numpy()[:] = np.asarray(segs_all, dtype=np.int64).reshape(-1, 4)
                my_table.copy_(my_table_host, non_blocking=True)
                pending.append(dist.isend(my_table, dst=0))
        for q in pending:
            q.wait()
        seg_info["segs"], seg_info["used"], seg_info["gathered"] = segs_all, used_total, at
        if timers:
            timers[1].record(stream)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # The workload description holds millions of Python objects (per-channel scale lists); a cyclic
    # garbage collection walking them would stall the host in the middle of a step.
    gc.collect()
    gc.freeze()
    sampler = ClockSampler(local_rank)
    sampler.start()  # sampled from the warm-up on: the timed region can be shorter than nvidia-smi's start-up
    for _ in range(max(args.warmup, 0)):
        step()
    sync_all()
    launches0 = backend.launch_count()
    def mk():
        return torch.cuda.Event(enable_timing=True)

    ev = [(mk(), mk(), [(mk(), mk(), mk()) for _ in cf]) for _ in range(args.steps)]
    t_begin, t_end = mk(), mk()
    t_begin.record(stream)
    seg_info["issue_s"] = 0.0
    for k in range(args.steps):
        step(ev[k])
    fold_issue_ms = seg_info["issue_s"] * 1e3 / max(1, args.steps)
    t_end.record(stream)
    sync_all()
    clocks = sampler.stop()
    launches = backend.launch_count() - launches0
    elapsed_ms = t_begin.elapsed_time(t_end)
    if world > 1:
        t = torch.tensor([elapsed_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
        ln = torch.tensor([launches], dtype=torch.int64, device="cuda")
        dist.all_reduce(ln)
        launches = int(ln.item())
    ms_per_step = elapsed_ms / args.steps
    live = [k for k, f in enumerate(cf) if f is not None]
    fold_ms = float(np.mean([sum(e[2][k][0].elapsed_time(e[2][k][1]) for k in live) for e in ev]))
    codec_ms = float(np.mean([sum(e[2][k][1].elapsed_time(e[2][k][2]) for k in live) for e in ev]))
    step_ms_local = float(np.mean([e[0].elapsed_time(e[1]) for e in ev]))
    gather_ms = max(0.0, step_ms_local - fold_ms - codec_ms)  # exposed (not hidden) part of the exchange
    per_rank = None
    if world > 1:  # every rank's own view of the timed region: [ms per step, fold, codec] on its stream
        mine_t = torch.tensor([t_begin.elapsed_time(t_end) / args.steps, fold_ms, codec_ms], dtype=torch.float64, device="cuda")
        all_t = [torch.zeros_like(mine_t) for _ in range(world)]
        dist.all_gather(all_t, mine_t)
        per_rank = [[round(float(x), 3) for x in t.tolist()] for t in all_t]

    # algorithmic bytes of the whole job (all ranks)
    stream_sizes = {i: sz for i, _, sz, comp in seg_info["segs"] if comp}
    fold_b, codec_b = algorithmic_bytes(mine, folder.folded_sizes, [stream_sizes.get(i) for i in range(len(mine))])
    blob_local = sum(sz for _, _, sz, _ in seg_info["segs"])
    tot = torch.tensor([fold_b, codec_b, sum(1 for _, _, _, c in seg_info["segs"] if c), blob_local],
                       dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(tot)
    fold_all, codec_all, n_compressed, blob_bytes = [float(x) for x in tot.tolist()]
    value = (fold_all + codec_all) / (ms_per_step * 1e-3) / 1e9

    # roofline of the dominant kernel: the fused fold pass, one launch per linear weight
    peak, peak_kind = measured_peak()
    # kernel launches of the fold phase (the batched entry point issues one launch per kernel
    # configuration and chunk, not one per tensor)
    l0 = backend.launch_count()
    for k, f in enumerate(cf):
        if f is not None:
            f.fold([in_ptrs[i] for i in chunks[k]], folded.data_ptr() + fold_off[k], True, [side[i] for i in chunks[k]])
    torch.cuda.synchronize()
    n_fold_launch = int(backend.launch_count() - l0)
    fold_local_b, _ = algorithmic_bytes(mine, folder.folded_sizes, [None] * len(mine))
    achieved = fold_local_b / (fold_ms * 1e-3) / 1e9 if fold_ms > 0 else 0.0
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None, "peak_kind": peak_kind, "kernel": "rowQuantRegBatchKernel (fused quantise + reorder + swizzle, all tensors of a configuration per launch)",
                "launches_per_step": n_fold_launch, "avg_launch_ms": fold_ms / max(1, n_fold_launch),
                "tensors_per_step": len([d for d in mine if d.transforms]),
                "algorithmic_bytes_per_launch": fold_local_b / max(1, n_fold_launch),
                "phase_ms": {"fold": fold_ms, "codec": codec_ms, "gather": gather_ms, "fold_host_issue": fold_issue_ms},
                "per_rank_ms": per_rank}
    if args.workload == "llama7b":
        # DRAM traffic of the dominant kernel from its ncu capture on the 2-layer case of this workload
        # (profiles/rowQuantRegBatchKernel_llama7b_2layers.md, first launch: 576.79 MB read + 259.20 MB
        # written for 576.72 MB + 288.36 MB + 0.56 MB of algorithmic bytes), scaled by the bytes of a launch:
        # traffic grows in proportion to the rows processed
        roofline["traffic"] = DRAM_PER_ALGORITHMIC_BYTE * roofline["algorithmic_bytes_per_launch"]
        roofline["traffic_source"] = "ncu capture of a smaller case, scaled by algorithmic bytes"

    # end to end through the C ABI with host buffers (pinned), copies inside the timed region.
    # The shard is processed in chunks of about 1.5 GB of input: while chunk c+1 uploads and folds on
    # the main stream, chunk c's segments (compressed, raw and pass-through) download on a second
    # stream, so both PCIe directions are busy.
    e2e = None
    if not args.no_e2e:
        host_in = [torch.empty(d.nbytes, dtype=torch.uint8, pin_memory=True) for d in mine]
        for h, t in zip(host_in, inputs):
            h.copy_(t)
        torch.cuda.synchronize()
        e_chunks, cur, cur_bytes = [], [], 0
        for i, d in enumerate(mine):
            if cur and cur_bytes + d.nbytes > 1_500_000_000:
                e_chunks.append(cur)
                cur, cur_bytes = [], 0
            cur.append(i)
            cur_bytes += d.nbytes
        if cur:
            e_chunks.append(cur)
        e_cf = [ShardFolder(backend, [mine[i] for i in c]) for c in e_chunks]
        e_fold_off, fo = [], 0
        for f in e_cf:
            e_fold_off.append(fo)
            fo += f.folded_bytes
        e_folded = torch.empty(fo, dtype=torch.uint8, device="cuda")
        host_blob = torch.empty(fo, dtype=torch.uint8, pin_memory=True)
        copy_stream = torch.cuda.Stream()

        def e2e_step():
            d2h = 0
            for k, (c, f) in enumerate(zip(e_chunks, e_cf)):
                f.fold([host_in[i].data_ptr() for i in c], e_folded.data_ptr() + e_fold_off[k], False,
                       [side[i] for i in c], max_batch_bytes=1 << 30)
                segs = f.compress_inplace(e_folded.data_ptr() + e_fold_off[k])
                done = torch.cuda.Event()
                done.record(stream)
                copy_stream.wait_event(done)
                with torch.cuda.stream(copy_stream):
                    for j, off, sz, _ in segs:  # each constant's bytes (stream or folded) go home
                        a = e_fold_off[k] + off
                        host_blob[a:a + sz].copy_(e_folded[a:a + sz], non_blocking=True)
                        d2h += sz
            stream.wait_stream(copy_stream)
            return d2h

        e2e_step()
        sync_all()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        d2h_bytes = 0
        for _ in range(max(1, args.e2e_steps)):
            d2h_bytes = e2e_step()
        b.record(stream)
        sync_all()
        ems = a.elapsed_time(b) / max(1, args.e2e_steps)
        if world > 1:
            t = torch.tensor([ems], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ems = float(t.item())
        h2d = torch.tensor([sum(d.nbytes for d in mine), d2h_bytes], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(h2d)
        e2e = {"value": (fold_all + codec_all) / (ems * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ems,
               "h2d_bytes_per_step": int(h2d[0].item()), "d2h_bytes_per_step": int(h2d[1].item()),
               "chunks": len(e_chunks)}
        del host_in, host_blob, e_folded

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        gbs, ms, cores, desc = run_cpu(decls, 1, 1, args.cpu_sample_elements)  # one untimed pass first: page faults, thread start-up
        cpu = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": desc, "ms_per_sample": ms}

    if rank == 0:
        line = {"metric": "folded_weight_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": dtype_name, "data": "synthetic", "config": config, "clocks": clocks,
                "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline, "cpu_baseline": cpu,
                "bytes": {"fold": fold_all, "codec": codec_all, "blob": blob_bytes, "compressed_tensors": n_compressed},
                "per_gpu_GBps": value / world}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
