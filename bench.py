#!/usr/bin/env python
"""Benchmark of the ruy::Mul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload `c3_i8`: the large projection, 4096 x 4096 int8 weights (prepacked, resident)
times 4096 x 8192 int8 activations -> int8 with per-row multipliers, bias, zero point and clamp.
One step = one such mul.  With N > 1 (launched under torchrun, one rank per GPU) the 8192
columns are sharded over the ranks and the destination shards are all-gathered over NCCL inside
the timed step (strong scaling).  Prints one JSON line on rank 0.

`--impl reference` times ruy's own CPU path (the compiled reference under oracle/_ref when
present, else the C port of the oracle) on the host cores on a bounded sample of the workload.
"""
import argparse
import ctypes as C
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "int8_gemm_tops"
UNIT = "TOP/s"
L2_FLUSH_BYTES = 256 << 20


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only queries) every few milliseconds
    from a host thread; `mark()` brackets the timed region so that only samples taken during it are
    summarised (all samples since start() if the region was too short to catch three)."""

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.samples = []   # (t, sm_mhz, reasons_bitmask)
        self.t0 = self.t1 = None
        self.stop_flag = False
        self.thread = None
        self.max_mhz = None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(gpu_index))
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self._reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
        except Exception as e:  # NVML missing: report that rather than guess
            self.nv = None
            self.err = str(e)

    @staticmethod
    def _physical_index(local_index):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if local_index < len(ids) and ids[local_index].isdigit():
                return int(ids[local_index])
        return local_index

    def start(self):
        if self.nv is None:
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                reasons = self._reasons(self.handle)
                self.samples.append((time.perf_counter(), float(mhz), int(reasons)))
            except Exception:
                pass
            time.sleep(0.002)

    def mark_begin(self):
        self.t0 = time.perf_counter()

    def mark_end(self):
        self.t1 = time.perf_counter()

    def stop(self):
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable: " + getattr(self, "err", "")]}
        self.stop_flag = True
        self.thread.join(timeout=2)
        nv = self.nv
        inside = [x for x in self.samples if self.t0 is not None and self.t0 <= x[0] <= (self.t1 or 1e30)]
        window = "timed region"
        if len(inside) < 3:
            inside, window = self.samples, "warm-up + timed region"
        bits = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
        reasons = sorted(name for name, bit in bits.items() if any(x[2] & bit for x in inside))
        return {"sm_mhz": float(np.median([x[1] for x in inside])) if inside else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(inside), "window": window}


def host_cpu():
    """Model name, logical CPUs and physical cores of this host, from /proc/cpuinfo."""
    model, cores, logical = "unknown", set(), 0
    try:
        phys = core = None
        for line in open("/proc/cpuinfo"):
            key, _, val = line.partition(":")
            key, val = key.strip(), val.strip()
            if key == "processor":
                logical += 1
            elif key == "model name":
                model = val
            elif key == "physical id":
                phys = val
            elif key == "core id":
                core = val
                cores.add((phys, core))
    except OSError:
        pass
    logical = logical or (os.cpu_count() or 1)
    return {"cpu_model": model, "logical_cpus": logical, "physical_cores": len(cores) or logical}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ------------------------------------------------------------------------------------------
# CPU arms
# ------------------------------------------------------------------------------------------

class CpuArm:
    """ruy's own CPU implementation of the workload on the host cores: the compiled reference (oracle/_ref) runs the
    FULL 4096 x 4096 x 8192 mul with the weights in ruy's prepacked cache, on every logical CPU.  Without the
    compiled reference the scalar C port of the oracle runs a small slice on one thread."""

    def __init__(self, workload):
        import oracle
        from ruy_b200 import cases
        from ruy_b200.api import make_desc
        self.oracle = oracle
        self.ref = oracle.reference()
        self.host = host_cpu()
        dst = "int32" if workload == "c3_i32" else "int8"
        if self.ref is not None:
            self.case = cases.config3(dst=dst)
            self.cores = self.host["logical_cpus"]
            self.kind = "reference"
            self.ctx = self.ref.ruy_ref_ctx_create(oracle.host_simd_path(), self.cores)
            self.same_config = True
        else:
            self.case = cases.config3(rows=512, depth=4096, cols=64, dst=dst)
            self.cores = 1
            self.kind = "port"
            self.ctx = None
            self.same_config = False
        self.dst = self.case.new_dst()
        self.bound = self.case.bind(self.dst)
        self.desc = make_desc(self.bound[0], self.bound[1], self.bound[2], self.bound[3])
        self.sample = f"{self.case.rows}x{self.case.depth} weights x {self.case.cols} of 8192 columns"

    def seconds(self, windows=1, min_secs=0.0):
        """Best seconds per mul over `windows` windows of at least `min_secs` (ruy/test.h:2082-2136)."""
        if self.ref is not None:
            return self.ref.ruy_ref_time_mul(self.ctx, C.byref(self.desc), windows, min_secs)
        t0 = time.perf_counter()
        self.oracle.oracle().ruy_oracle_mul(C.byref(self.desc), 1, 0)
        return time.perf_counter() - t0

    def describe(self):
        if self.ref is not None:
            used = {0x40: "kAvx512", 0x20: "kAvx2Fma", 0x10: "kAvx", 0x1: "kStandardCpp"}.get(
                self.ref.ruy_ref_last_used_path(self.ctx), "?")
            return (f"{self.sample} (the whole mul); ruy::Mul on {used}, {self.cores} threads on {self.host['physical_cores']} "
                    f"physical cores of {self.host['cpu_model']}, weights in the prepacked cache")
        return f"{self.sample}; scalar C port of the oracle, 1 thread"

    def baseline(self, value, unit=UNIT):
        return {"value": value, "unit": unit, "cores": self.cores, "physical_cores": self.host["physical_cores"],
                "cpu_model": self.host["cpu_model"], "kind": self.kind, "sample": self.describe()}

    def tops(self, secs):
        return self.case.ops / secs / 1e12

    def close(self):
        if self.ctx is not None:
            self.ref.ruy_ref_ctx_destroy(self.ctx)
            self.ctx = None


def run_reference_arm(args):
    rank, world, local = dist_env()
    if rank != 0:
        return
    arm = CpuArm(args.workload)
    for _ in range(max(args.warmup, 1)):
        arm.seconds()
    secs = [arm.seconds() for _ in range(args.steps)]
    ms = float(np.mean(secs)) * 1e3
    value = arm.tops(float(np.mean(secs)))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": {"workload": args.workload, "rows": 4096, "depth": 4096, "cols": 8192,
                   "same_config": arm.same_config,
                   "note": "each step is the whole mul on the host cores" if arm.same_config else
                           "each step times one bounded sample of the workload on the host cores"},
        "cpu_baseline": arm.baseline(value),
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    arm.close()
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel of each workload on one
# GPU, from ncu captures of this benchmark; a capture cannot run inside a timed benchmark, so the figure is carried
# here with the commit it was taken at.
NCU_TRAFFIC = {
    "c3_i8": {"bytes": 51.7e6, "source": "ncu launch list of `bench.py --steps 3 --warmup 3 --no-sustained --no-cpu-baseline`, captured at commit d076546"},
    "c2": {"bytes": 193.3e6, "source": "ncu capture of `bench.py --workload c2 --steps 3 --warmup 3 --no-cpu-baseline`, captured at commit d076546"},
}
NOMINAL_INT8_TOPS = 4500.0   # B200 dense int8, vendor figure


def pinned_copy_peak(dev, torch):
    """GB/s per direction of 64 MiB pinned-memory copies running in both directions at once (the pattern of the
    end-to-end step), best of 5."""
    n = 64 << 20
    h_in = torch.empty(n, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(n, dtype=torch.uint8).pin_memory()
    d_in = torch.empty(n, dtype=torch.uint8, device=dev)
    d_out = torch.empty(n, dtype=torch.uint8, device=dev)
    s1, s2 = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    best = 0.0
    for _ in range(5):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        with torch.cuda.stream(s1):
            d_in.copy_(h_in, non_blocking=True)
        with torch.cuda.stream(s2):
            h_out.copy_(d_out, non_blocking=True)
        torch.cuda.synchronize()
        best = max(best, n / (time.perf_counter() - t0) / 1e9)
    return best


def verify_small_muls(mine, host_dst, dst_off, rounding, what):
    """Every destination of a list of small MulCases against the CPU oracle (host threads; the C library releases
    the interpreter lock).  Raises SystemExit on the first difference; returns the number of muls checked."""
    from concurrent.futures import ThreadPoolExecutor
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import util

    def check(i):
        c = mine[i]
        got = c.dst_view(host_dst[dst_off[i]:dst_off[i] + c.dst_storage_elems()])
        return i if not np.array_equal(got, util.run_oracle(c, rounding)) else -1

    with ThreadPoolExecutor(max_workers=min(32, os.cpu_count() or 1)) as pool:
        bad = [i for i in pool.map(check, range(len(mine))) if i >= 0]
    if bad:
        raise SystemExit(f"bench.py: {len(bad)} of {len(mine)} {what} do not match the oracle (first: {bad[:4]}); refusing to report")
    return len(mine)


def measure_c2(args, torch, dev, rank, world, local, dist):
    """Batched small muls (config 2): 16384 independent int8 muls with dims drawn from {16..128}, weights in the
    prepacked cache, one plan replayed per step with a single persistent launch.  With N ranks the mul index
    range is split evenly (no collective: the destinations stay where their consumers are).  Returns the record."""
    import ruy_b200
    from ruy_b200 import _abi, cases
    from ruy_b200.api import CachePolicy, Matrix, MulParams, Rounding
    from ruy_b200.sharding import mul_range
    use_dist = world > 1
    n_total = args.muls
    first, count = mul_range(n_total, rank, world)
    mine = cases.config2(n=n_total, seed=0, first=first, count=count)

    def pool(arrays, dtype):
        """One device buffer holding all arrays at 256-byte aligned offsets; returns (tensor, offsets)."""
        offs, total = [], 0
        item = np.dtype(dtype).itemsize
        for a in arrays:
            offs.append(total)
            total += (a.size * item + 255) // 256 * 256 // item
        host = np.zeros(max(total, 1), dtype=dtype)
        for a, o in zip(arrays, offs):
            host[o:o + a.size] = a
        return torch.from_numpy(host).to(dev), offs

    lhs_buf, lhs_off = pool([c.lhs for c in mine], np.int8)
    rhs_buf, rhs_off = pool([c.rhs for c in mine], np.int8)
    bias_buf, vec_off = pool([c.bias for c in mine], np.int32)
    mfp_buf, _ = pool([c.mfp for c in mine], np.int32)
    mexp_buf, _ = pool([c.mexp for c in mine], np.int32)
    dst_buf, dst_off = pool([c.new_dst() for c in mine], np.int8)

    stream = torch.cuda.Stream(device=dev)
    ctx = ruy_b200.Context(local, stream=stream.cuda_stream)
    descs = []
    for i, c in enumerate(mine):
        lhs = Matrix(lhs_buf[lhs_off[i]:], c.lhs_layout, c.lhs_zp, CachePolicy.kAlwaysCache)
        rhs = Matrix(rhs_buf[rhs_off[i]:], c.rhs_layout, c.rhs_zp)
        dst = Matrix(dst_buf[dst_off[i]:], c.dst_layout, c.dst_zp)
        p = MulParams("int32", "int8")
        p.bias = bias_buf[vec_off[i]:]
        p.multiplier_fixedpoint_perchannel = mfp_buf[vec_off[i]:]
        p.multiplier_exponent_perchannel = mexp_buf[vec_off[i]:]
        p.clamp_min, p.clamp_max = c.clamp
        p.rounding = Rounding.kReference
        descs.append(ruy_b200.make_desc(lhs, rhs, p, dst))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    plan = ruy_b200.Plan(ctx, descs)
    plan_build_s = time.perf_counter() - t0
    nbytes, ops = plan.stats()
    with torch.cuda.stream(stream):
        flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
        sampler = ClockSampler(local)
        sampler.start()
        for _ in range(max(args.warmup, 3)):
            flush.fill_(1)
            plan.run()
        ctx.sync()
        launches0 = ctx.counters()["launches"]
        if use_dist:
            dist.barrier()
        torch.cuda.synchronize()
        sampler.mark_begin()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        for i in range(args.steps):
            flush.fill_(i & 0xFF)
            starts[i].record(stream)
            plan.run()
            stops[i].record(stream)
        stream.synchronize()
        if use_dist:
            dist.barrier()
        torch.cuda.synchronize()
        sampler.mark_end()
        clocks = sampler.stop()
        launches = ctx.counters()["launches"] - launches0
        # parity: every destination of this rank's muls, as the timed replays left them
        checked = verify_small_muls(mine, dst_buf.cpu().numpy(), dst_off, Rounding.kReference, "small muls")
        ms = float(np.sum([a.elapsed_time(b) for a, b in zip(starts, stops)])) / args.steps
        if use_dist:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
            tb = torch.tensor([float(nbytes), float(ops), float(checked)], dtype=torch.float64, device=dev)
            dist.all_reduce(tb)
            total_bytes, total_ops, checked = float(tb[0]), float(tb[1]), int(tb[2])
        else:
            total_bytes, total_ops = float(nbytes), float(ops)
    peaks = measured_peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9     # this rank's bytes over the slowest rank's time: the per-GPU roofline figure
    known = NCU_TRAFFIC["c2"] if (world == 1 and n_total == 16384) else None
    line = {
        "metric": "small_mul_muls_per_s", "value": n_total / (ms * 1e-3), "unit": "muls/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "c2", "muls": n_total, "dims": list(cases.CONFIG2_DIMS),
                   "sharding": f"{world} shard(s) by mul index", "l2": f"flushed between steps ({L2_FLUSH_BYTES >> 20} MiB fill, untimed)",
                   "plan_build_s": plan_build_s},
        "gpu_launches": int(launches), "clocks": clocks, "checked_muls": checked,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                     "traffic": known["bytes"] if known else None, "traffic_source": known["source"] if known else None,
                     "kernel": "batch_i8_kernel", "algorithmic_bytes": nbytes,
                     "peak_source": f"hbm_gbs of {peaks['source']} peaks"},
        "tops": total_ops / (ms * 1e-3) / 1e12,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle
        ref = oracle.reference()
        if ref is not None:
            sample = cases.config2(n=n_total, seed=0, first=0, count=min(2048, n_total))
            keep, host_descs = [], (_abi.MulDesc * len(sample))()
            for i, c in enumerate(sample):
                b = c.bind(c.new_dst())
                keep.append(b)
                host_descs[i] = ruy_b200.make_desc(b[0], b[1], b[2], b[3])
            host = host_cpu()
            cores = host["logical_cpus"]
            secs = ref.ruy_ref_time_batch(host_descs, len(sample), cores, oracle.host_simd_path(), 5)
            line["cpu_baseline"] = {"value": len(sample) / secs, "unit": "muls/s", "cores": cores,
                                    "physical_cores": host["physical_cores"], "cpu_model": host["cpu_model"], "kind": "reference",
                                    "sample": f"first {len(sample)} of {n_total} muls; {cores} host threads, one ruy::Context each, "
                                              "LHS in ruy's prepacked cache"}
    plan.close()
    ctx.close()
    return line


def run_c2_arm(args):
    import torch
    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    line = measure_c2(args, torch, dev, rank, world, local, dist)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_gpu_arm(args):
    import torch
    import ruy_b200
    from ruy_b200 import cases
    from ruy_b200._lib import lib
    from ruy_b200.api import Rounding

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the GPU arm has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    use_dist = world > 1
    dist = None
    if use_dist:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    dst_name = "int32" if args.workload == "c3_i32" else "int8"
    from ruy_b200.sharding import column_shard
    cols_total = args.cols
    first_col, shard = column_shard(cols_total, rank, world)
    case = cases.config3(dst=dst_name, col_begin=first_col, col_count=shard)
    tdtype = torch.int32 if dst_name == "int32" else torch.int8
    esz = 4 if dst_name == "int32" else 1
    peaks = measured_peaks()

    stream = torch.cuda.Stream(device=dev)
    ctx = ruy_b200.Context(local, stream=stream.cuda_stream)
    mirrored = use_dist and args.gather == "mirror"
    flags = None
    gather_sets = {}     # how the shards reach every rank -> two gathered destination buffers, used by step parity
    if use_dist:
        from ruy_b200 import peer
    if mirrored:
        # Two gathered destinations per mode: a rank that has left its exchange may start the next step while a slower
        # peer still reads the previous one (see ruyb200_mul_async_mirrored_exchange).  "multicast": an NVLink multicast
        # mapping over every rank's buffer, a rank stores its shard once and the switch delivers it everywhere (not on
        # platforms without such mappings, nor with RUYB200_BENCH_MULTICAST=0); "peer_stores": the epilogue stores to
        # each peer's buffer.  Which of the two is faster depends on the number of ranks; a short trial below decides.
        nbytes = cols_total * case.rows * esz
        if esz == 1 and os.environ.get("RUYB200_BENCH_MULTICAST", "1") != "0":
            bufs = None
            try:
                bufs = [peer.MulticastBuffer(nbytes, dev) for _ in range(2)]
            except Exception as e:
                if rank == 0:
                    print(f"bench.py: no multicast mapping ({type(e).__name__}: {str(e)[:120]})", file=sys.stderr)
            ok = torch.tensor([1 if bufs else 0], dtype=torch.int32, device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok[0]) == 1:
                gather_sets["multicast"] = bufs
            elif bufs:
                for b in bufs:
                    b.close()
        if os.environ.get("RUYB200_BENCH_MULTICAST", "1") != "only" or not gather_sets:
            gather_sets["peer_stores"] = [peer.PeerBuffer(nbytes, dev) for _ in range(2)]
        flags = peer.StepFlags(dev)
    shard_elems = shard * case.rows
    shard_bytes = shard_elems * esz
    # even / odd steps are told apart by the destination zero point (5 / 6): every unsaturated output differs by one
    tag = (lambda par: par) if dst_name == "int8" else (lambda par: 0)
    with torch.cuda.stream(stream):
        G = {}     # the gather mode in use: its buffers and the views and addresses derived from them

        def use_gather(name):
            bufs = gather_sets.get(name, [])
            G["name"], G["bufs"] = name, bufs
            G["fulls"] = ([b.tensor.view(tdtype) for b in bufs] if mirrored
                          else [torch.zeros(cols_total * case.rows, dtype=tdtype, device=dev)])
            G["mines"] = [f[rank * shard_elems:(rank + 1) * shard_elems] for f in G["fulls"]]
            G["dsts"] = [ruy_b200.Matrix(m, case.dst_layout, case.dst_zp + tag(par)) for par, m in enumerate(G["mines"])]
            G["mirror_ptrs"] = [[q + rank * shard_bytes for r_, q in enumerate(b.ptrs) if r_ != rank] for b in bufs]

        use_gather(next(iter(gather_sets)) if gather_sets else None)
        lhs, rhs, p, d0, keep = case.bind(G["mines"][0], device=dev, rounding=Rounding.kReference)
        flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
        ruy_b200.mul(lhs, rhs, p, ctx, G["dsts"][0])  # packs the weights into the context's device cache
        # With four or more ranks a shard is one or two rounds of 256 x 256 tiles, and a tile's stores can only start when
        # its whole depth is done: a second context with 256 x 128 tiles (more rounds, stores start earlier, slower
        # kernel) takes part in the trial below.
        tile_ctxs = {"": ctx}
        if mirrored and world >= 4 and not os.environ.get("RUYB200_TILE"):
            os.environ["RUYB200_TILE"] = "pair:128"
            try:
                tile_ctxs["pair:128"] = ruy_b200.Context(local, stream=stream.cuda_stream)
            finally:
                del os.environ["RUYB200_TILE"]
            ruy_b200.mul(lhs, rhs, p, tile_ctxs["pair:128"], G["dsts"][0])
        G["ctx"], G["tile"] = ctx, ""
        step_no = [0]

        def plain_step(gather):
            ruy_b200.mul_async(lhs, rhs, p, ctx, G["dsts"][0])
            if gather:
                dist.all_gather_into_tensor(G["fulls"][0], G["mines"][0])

        def fused_step():
            step_no[0] += 1
            par = step_no[0] & 1
            # the epilogue stores each tile here and in every peer's buffer, and the launch ends with the flag exchange
            if G["name"] == "multicast":
                peer.mul_async_multicast(lhs, rhs, p, G["ctx"], G["dsts"][par], G["bufs"][par].multicast_ptr + rank * shard_bytes,
                                         flags, step_no[0])
            else:
                peer.mul_async_mirrored(lhs, rhs, p, G["ctx"], G["dsts"][par], G["mirror_ptrs"][par], flags=flags, value=step_no[0])

        def timed(fn, steps):
            """`steps` calls of fn, each between its own event pair after an untimed L2 flush; max over ranks of the mean ms."""
            for _ in range(3):
                flush.fill_(1)
                fn()
            stream.synchronize()
            if use_dist:
                dist.barrier()
            torch.cuda.synchronize()
            starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
            stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
            for i in range(steps):
                flush.fill_(i & 0xFF)          # evict the operands from L2 (not timed)
                starts[i].record(stream)
                fn()
                stops[i].record(stream)
            stream.synchronize()
            if use_dist:
                dist.barrier()
            torch.cuda.synchronize()
            ms = float(np.mean([s.elapsed_time(e) for s, e in zip(starts, stops)]))
            if use_dist:
                t = torch.tensor([ms], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t[0])
            return ms

        main_step = fused_step if mirrored else (lambda: plain_step(use_dist))
        gather_trial = {}
        if len(gather_sets) * len(tile_ctxs) > 1:
            # five steps of each mode and tile shape (the time is the max over ranks, so every rank takes the same decision)
            combos = [(name, tile) for name in gather_sets for tile in tile_ctxs]
            for name, tile in combos:
                use_gather(name)
                G["ctx"], G["tile"] = tile_ctxs[tile], tile
                gather_trial[name + (" " + tile if tile else "")] = timed(fused_step, 5)
            best = min(range(len(combos)), key=lambda i: list(gather_trial.values())[i])
            use_gather(combos[best][0])
            G["ctx"], G["tile"] = tile_ctxs[combos[best][1]], combos[best][1]
        sampler = ClockSampler(local)
        sampler.start()
        for _ in range(max(args.warmup, 3)):
            flush.fill_(1)
            main_step()
        stream.synchronize()

        rs = np.arange(0, case.rows, 509)
        cs = np.arange(0, shard, 211)
        Lrows = case.lhs.reshape(case.rows, case.depth).astype(np.int64)[rs]

        def expected(c, par, ncols=None, cols_sel=None):
            ncols = shard if ncols is None else ncols
            cols_sel = cs if cols_sel is None else cols_sel
            acc = Lrows @ c.rhs.reshape(ncols, case.depth).astype(np.int64)[cols_sel].T
            if dst_name == "int8":
                acc = acc + case.bias.astype(np.int64)[rs][:, None]
                m, e = case.mfp.astype(np.int64)[rs][:, None], case.mexp.astype(np.int64)[rs][:, None]
                acc = np.clip(((acc * m + (1 << (30 - e))) >> (31 - e)) + case.dst_zp + tag(par), -128, 127)
            return acc

        nb = (rank + 1) % world
        nb_case = cases.config3(dst=dst_name, col_begin=nb * shard, col_count=shard) if use_dist else None

        def leave_together(problem):
            """A failed check ends the run on every rank at the same point and in order (buffers unbound after a barrier,
            nobody left waiting in a collective): a rank must not disappear while its memory is part of a mapping that
            its peers still store into."""
            if use_dist:
                t = torch.tensor([1 if problem else 0], dtype=torch.int32, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                if int(t[0]) == 0:
                    return
                stream.synchronize()
                if mirrored:
                    flags.close()
                    for bufs in gather_sets.values():
                        for b in bufs:
                            b.close()
                dist.barrier()
                raise SystemExit(problem or "bench.py: another rank found a wrong result; refusing to report")
            if problem:
                raise SystemExit(problem)

        def check_buffers(when):
            """Sampled sub-blocks of this rank's shard and of the next rank's shard as gathered here, in every
            destination buffer, against 64-bit numpy arithmetic."""
            problem = None
            for par, f in enumerate(G["fulls"]):
                out = case.dst_view(f[rank * shard_elems:(rank + 1) * shard_elems].cpu().numpy())
                if not np.array_equal(out[np.ix_(rs, cs)].astype(np.int64), expected(case, par)):
                    problem = f"bench.py: GPU result does not match the reference arithmetic ({when}); refusing to report"
                if use_dist:
                    nb_out = nb_case.dst_view(f[nb * shard_elems:(nb + 1) * shard_elems].cpu().numpy())
                    if not np.array_equal(nb_out[np.ix_(rs, cs)].astype(np.int64), expected(nb_case, par)):
                        problem = f"bench.py: the gathered destination is wrong ({when}); refusing to report"
            leave_together(problem)

        if mirrored and (step_no[0] & 1) == 0:
            fused_step()      # so that both buffers have been written
            stream.synchronize()
        check_buffers("after warm-up")

        launches0 = G["ctx"].counters()["launches"]
        if use_dist:
            dist.barrier()
        torch.cuda.synchronize()
        sampler.mark_begin()
        wall0 = time.perf_counter()
        ms_per_step = timed(main_step, args.steps)
        wall = time.perf_counter() - wall0
        sampler.mark_end()
        clocks = sampler.stop()
        launches = G["ctx"].counters()["launches"] - launches0 - 3     # `timed` runs three untimed calls first
        check_buffers("after the timed steps")
        total_ops = 2.0 * case.rows * case.depth * cols_total
        value = total_ops / (ms_per_step * 1e-3) / 1e12
        # the kernel alone, destination left where it is computed (at N = 1 this is the step itself)
        kernel_ms = timed(lambda: plain_step(False), args.steps) if use_dist else ms_per_step
        variants = {"kernel_only_tops": total_ops / (kernel_ms * 1e-3) / 1e12}
        if use_dist:
            nccl_ms = timed(lambda: plain_step(True), args.steps)
            variants["gather_nccl_tops"] = total_ops / (nccl_ms * 1e-3) / 1e12
            variants["gather_fused_tops"] = value if mirrored else None
            variants["value_is"] = "gather_fused_tops" if mirrored else "gather_nccl_tops"
            if mirrored:
                variants["gather_mode"] = G["name"] + (", tiles " + G["tile"] if G["tile"] else "")
                if gather_trial:
                    variants["gather_trial_ms"] = gather_trial
            variants["note"] = ("strong scaling of one 4096x4096x8192 mul: every rank must receive (N-1)/N of the 33.6 MB "
                                "destination, so the gather-inclusive step is bounded by NVLink ingress, not by the math")
            # Weak scaling beside it: the benchmark's whole mul on every rank (its own 8192 activation columns of an
            # 8192 x N column problem, same weights), destination left sharded, no exchange: the data-parallel reading.
            wcase = cases.config3(dst=dst_name, col_begin=rank * cols_total, col_count=cols_total)
            wdst = torch.zeros(wcase.dst_storage_elems(), dtype=tdtype, device=dev)
            wl, wr, wp, wd, wkeep = wcase.bind(wdst, device=dev, rounding=Rounding.kReference)
            ruy_b200.mul(wl, wr, wp, ctx, wd)
            weak_ms = timed(lambda: ruy_b200.mul_async(wl, wr, wp, ctx, wd), args.steps)
            wcs = np.arange(0, cols_total, 997)
            wout = wcase.dst_view(wdst.cpu().numpy())[np.ix_(rs, wcs)].astype(np.int64)
            leave_together(None if np.array_equal(wout, expected(wcase, 0, cols_total, wcs)) else
                           "bench.py: weak-scaling result does not match the reference arithmetic; refusing to report")
            variants["weak"] = {"cols_per_rank": cols_total, "ms_per_step": weak_ms,
                                "tops": world * 2.0 * case.rows * case.depth * cols_total / (weak_ms * 1e-3) / 1e12,
                                "note": "every rank multiplies the same weights by its own 8192 activation columns; "
                                        "destination left sharded, no exchange"}
            del wdst, wkeep

        # sustained: at least a second of back-to-back muls over four rotating activation / destination sets (268 MB, more
        # than L2), compared with the sustained (power-capped) peak
        sustained = None
        if not use_dist and not args.no_sustained:
            sets = []
            for i in range(4):
                dd = torch.zeros(case.dst_storage_elems(), dtype=tdtype, device=dev)
                l2, r2, p2, d2, k2 = case.bind(dd, device=dev, rounding=Rounding.kReference)
                l2.data, p2.bias = lhs.data, p.bias
                p2.multiplier_fixedpoint_perchannel = p.multiplier_fixedpoint_perchannel
                p2.multiplier_exponent_perchannel = p.multiplier_exponent_perchannel
                sets.append((ruy_b200.make_desc(l2, r2, p2, d2), dd, k2, l2, r2, p2, d2))
            fn = lib().ruyb200_mul_async
            reps = max(64, int(1.2 / (ms_per_step * 1e-3)))
            for s_ in sets:
                fn(ctx._h, C.byref(s_[0]))
            stream.synchronize()
            s2 = ClockSampler(local)
            s2.start()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s2.mark_begin()
            e0.record(stream)
            for i in range(reps):
                fn(ctx._h, C.byref(sets[i & 3][0]))
            e1.record(stream)
            stream.synchronize()
            s2.mark_end()
            sclk = s2.stop()
            sus_ms = e0.elapsed_time(e1) / reps
            sus_tops = total_ops / (sus_ms * 1e-3) / 1e12
            sustained = {"tops": sus_tops, "ms_per_mul": sus_ms, "muls": reps, "seconds": sus_ms * reps * 1e-3,
                         "peak": 2.0 * peaks["bf16_tflops_sustained"], "frac": sus_tops / (2.0 * peaks["bf16_tflops_sustained"]),
                         "peak_source": f"2 x bf16_tflops_sustained of {peaks['source']} peaks",
                         "clocks": sclk, "l2": "four rotating activation/destination sets, 268 MB"}
            del sets

        # end to end through the public synchronous call with HOST buffers (weights stay cached)
        host_dst = case.new_dst()
        hl, hr, hp, hd, hkeep = case.bind(host_dst, rounding=Rounding.kReference)
        pinned_rhs = torch.from_numpy(case.rhs).pin_memory()
        pinned_dst = torch.empty(case.dst_storage_elems(), dtype=tdtype).pin_memory()
        hr.data, hd.data = pinned_rhs, pinned_dst
        # per-channel vectors and bias are host arrays as well
        ruy_b200.mul(hl, hr, hp, ctx, hd)
        c0 = ctx.counters()
        e2e_steps = max(2, min(args.steps, 10))
        if use_dist:
            dist.barrier()
        torch.cuda.synchronize()
        ruy_b200.mul(hl, hr, hp, ctx, hd)       # a second untimed call: the scratch arena has its final size only now
        c0 = ctx.counters()
        torch.cuda.synchronize()
        per_call = []
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            t1 = time.perf_counter()
            ruy_b200.mul(hl, hr, hp, ctx, hd)
            per_call.append((time.perf_counter() - t1) * 1e3)
        torch.cuda.synchronize()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        c1 = ctx.counters()
        if use_dist:
            t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_s = float(t[0])
        e2e_value = total_ops / e2e_s / 1e12
        h2d = (c1["h2d_bytes"] - c0["h2d_bytes"]) // e2e_steps
        d2h = (c1["d2h_bytes"] - c0["d2h_bytes"]) // e2e_steps
        if not np.array_equal(case.dst_view(pinned_dst.numpy())[np.ix_(rs, cs)].astype(np.int64), expected(case, 0)):
            leave_together("bench.py: end-to-end result mismatch")
        elif use_dist:
            leave_together(None)
        copy_peak = pinned_copy_peak(dev, torch)
        e2e_gbs = max(h2d, d2h) / e2e_s / 1e9

    # tcgen05 kind::i8 issues twice the multiply-adds per clock of kind::f16: the int8 dense peak is
    # taken as 2 x the measured dense bf16 throughput (the burst figure: the kernel is timed alone).
    peak_tops = 2.0 * peaks["bf16_tflops"]
    shard_ops = 2.0 * case.rows * case.depth * shard
    achieved = shard_ops / (kernel_ms * 1e-3) / 1e12
    known = NCU_TRAFFIC["c3_i8"] if (world == 1 and cols_total == 8192 and dst_name == "int8") else None
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak_tops, "unit": "TFLOP/s",
                "frac": achieved / peak_tops, "frac_of_nominal_int8_peak": achieved / NOMINAL_INT8_TOPS,
                "traffic": known["bytes"] if known else None, "traffic_source": known["source"] if known else None,
                "kernel": "tc_i8_kernel",
                "peak_source": f"2 x bf16_tflops of {peaks['source']} peaks; ops are int8 multiply-adds x 2",
                "kernel_ms": kernel_ms}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": {"workload": args.workload, "rows": case.rows, "depth": case.depth, "cols": cols_total,
                   "dst": dst_name,
                   "sharding": f"{world} column shard(s) of {shard}" + (
                       (", dst gathered on every rank inside the step by " +
                        (("one multimem store per piece into an NVLink multicast mapping of every rank's buffer" if G["name"] == "multicast"
                          else "epilogue stores into each peer's memory over NVLink") +
                         ", flag exchange inside the same launch, two destination buffers used by step parity"
                         if mirrored else "an NCCL all-gather"))
                       if use_dist else ""),
                   "l2": f"flushed between steps ({L2_FLUSH_BYTES >> 20} MiB fill, untimed)"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "ms_per_step": e2e_s * 1e3, "ms_per_call_min_max": [min(per_call), max(per_call)],
                "roofline": {"bound": "pcie", "achieved": e2e_gbs, "peak": copy_peak, "unit": "GB/s per direction",
                             "frac": e2e_gbs / copy_peak if copy_peak else None,
                             "peak_source": "64 MiB pinned copies in both directions at once, measured in this run"}},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": roofline,
        "wall_s": wall,
    }
    if use_dist:
        line["e2e"]["note"] = (f"each of the {world} ranks moves its own column shard over its own PCIe link (bytes per step are "
                               "one rank's); the destination stays in host memory as one slice per rank, it is not gathered")
    line.update(variants)
    if sustained:
        line["sustained"] = sustained
    ctx.sync()
    if mirrored:
        flags.close()
        for bufs in gather_sets.values():
            for b in bufs:
                b.close()
    for t, c in tile_ctxs.items():
        if t:
            c.sync()
            c.close()
    ctx.close()
    G.clear()
    del flush
    torch.cuda.empty_cache()
    # the small-mul half of the metric, in the same process: 16384 small muls as one plan, sharded by mul index
    if not args.no_c2:
        c2 = measure_c2(args, torch, dev, rank, world, local, dist)
        line["c2"] = {"metric": c2["metric"], "muls_per_s": c2["value"], "ms_per_step": c2["ms_per_step"], "muls": c2["config"]["muls"],
                      "plan_build_s": c2["config"]["plan_build_s"], "gpu_launches": c2["gpu_launches"], "checked_muls": c2["checked_muls"],
                      "roofline": c2["roofline"], "clocks": c2["clocks"], "cpu_baseline": c2.get("cpu_baseline"),
                      "sharding": c2["config"]["sharding"]}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        arm = CpuArm(args.workload)
        secs = arm.seconds(windows=4, min_secs=0.5 if arm.kind == "reference" else 0.0)
        line["cpu_baseline"] = arm.baseline(arm.tops(secs))
        arm.close()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if use_dist:
        dist.destroy_process_group()


def verify_case(case, got):
    """Checks a whole result: the CPU oracle for small cases, the compiled reference for large ones (sampled numpy
    arithmetic when that is absent).  Returns a word for the record; raises SystemExit on a difference."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import util
    from ruy_b200 import _abi
    import oracle
    if case.accum == "float32":
        wide = util.run_oracle(case, wide_float=True).astype(np.float64)
        if not np.all(np.abs(got.astype(np.float64) - wide) <= 1e-5 * np.maximum(np.abs(wide), 1.0)):
            raise SystemExit(f"bench.py: {case.name} is outside 1e-5 of the double-precision reference; refusing to report")
        return "oracle (float64 accumulation), 1e-5 relative"
    if case.ops <= 4e8:
        if not np.array_equal(got, util.run_oracle(case)):
            raise SystemExit(f"bench.py: {case.name} does not match the oracle; refusing to report")
        return "oracle, bit-exact"
    if oracle.reference() is not None:
        want = util.run_reference(case, path=_abi.PATH_STANDARD_CPP, threads=os.cpu_count() or 1)
        if not np.array_equal(got, want):
            raise SystemExit(f"bench.py: {case.name} does not match ruy's reference path; refusing to report")
        return "compiled reference (kStandardCpp), bit-exact"
    rng = np.random.default_rng(0)
    rs = np.sort(rng.choice(case.rows, min(case.rows, 64), replace=False))
    cs = np.sort(rng.choice(case.cols, min(case.cols, 256), replace=False))
    L = case.lhs.reshape(case.rows, case.depth).astype(np.int64)[rs]
    R = case.rhs.reshape(case.cols, case.depth).astype(np.int64)[cs]
    acc = (L - case.lhs_zp) @ (R - case.rhs_zp).T + case.bias.astype(np.int64)[rs][:, None]
    m, e = np.int64(case.mfp), np.int64(case.mexp)
    acc = np.clip(((acc * m + (np.int64(1) << (30 - e))) >> (31 - e)) + case.dst_zp, case.clamp[0], case.clamp[1])
    if not np.array_equal(got[np.ix_(rs, cs)].astype(np.int64), acc):
        raise SystemExit(f"bench.py: {case.name} does not match the reference arithmetic; refusing to report")
    return "sampled 64 x 256 block against 64-bit numpy, bit-exact"


def run_small_arm(args):
    """The remaining benchmark configurations, one JSON line each (single GPU, device-resident operands): config 0
    (256x512x128 int8), config 1 (the five fp32 shapes) and config 4 (the uint8 pointwise-conv layers at batch 1
    and 64); workload "narrow" adds config 3's weights against 1, 8 and 16 activation columns (one pass over the
    weights per mul, HBM-bound).  Timing follows ruy's cold protocol (ruy/test.h:2054-2080): the activations and the destination rotate
    over enough copies to exceed L2 (at least 256 MB, at most 48 copies), one pass over the copies through the
    stream-ordered entry point is captured in a CUDA graph, and several replays run between ONE pair of events, so
    neither the event overhead nor a cache flush is inside the figure.  Every result is checked before its line is
    printed.  Every line carries the same mul timed through ruy's own CPU path on all host cores."""
    import torch
    import ruy_b200
    from ruy_b200 import cases
    from ruy_b200._lib import lib
    from ruy_b200.api import Rounding, make_desc
    import oracle

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream(device=dev)
    ctx = ruy_b200.Context(0, stream=stream.cuda_stream)
    peaks = measured_peaks()
    todo = []
    if args.workload in ("c0", "small"):
        todo.append(cases.config0())
    if args.workload in ("c1", "small"):
        todo.extend(cases.config1(sh) for sh in cases.CONFIG1_SHAPES)
    if args.workload in ("c4", "small"):
        for batch in (1, 64):
            todo.extend(cases.config4(layer, batch=batch) for layer in range(len(cases.CONFIG4_LAYERS)))
    if args.workload == "narrow":
        # config 3's generator with a handful of columns: a weight matrix streamed once per mul (the narrow kernels)
        for rows, cols in ((4096, 1), (4096, 8), (16384, 1), (16384, 8), (16384, 16)):
            todo.append(cases.config3(rows=rows, depth=rows, cols=cols, dst="int8"))
    if args.only:
        todo = [c for c in todo if args.only in c.name]
        if not todo:
            raise SystemExit(f"bench.py: --only {args.only!r} matches no case of workload {args.workload}")
    ref = oracle.reference()
    host = host_cpu()
    cores = host["logical_cpus"]
    ref_ctx = ref.ruy_ref_ctx_create(oracle.host_simd_path(), cores) if ref is not None else None
    torch_dt = {"int8": torch.int8, "uint8": torch.uint8, "int32": torch.int32, "float32": torch.float32}
    fn = lib().ruyb200_mul_async
    with torch.cuda.stream(stream):
        for case in todo:
            nbytes = case.algorithmic_bytes()
            copies = int(max(2, min(48, ((256 << 20) + nbytes - 1) // nbytes)))
            sets, descs, first = [], [], None
            for i in range(copies):
                dst = torch.zeros(case.dst_storage_elems(), dtype=torch_dt[case.dst_dtype], device=dev)
                lhs, rhs, p, d, keep = case.bind(dst, device=dev, rounding=Rounding.kReference)
                if first is None:
                    first = (lhs, p)
                else:   # the weights and the per-channel vectors are shared; activations and destination rotate
                    lhs.data, p.bias = first[0].data, first[1].bias
                    p.multiplier_fixedpoint_perchannel = first[1].multiplier_fixedpoint_perchannel
                    p.multiplier_exponent_perchannel = first[1].multiplier_exponent_perchannel
                sets.append((dst, keep, lhs, rhs, p, d))
                descs.append(make_desc(lhs, rhs, p, d))
            for dsc in descs:      # warm-up; every one-time set-up happens here, outside the capture
                if fn(ctx._h, C.byref(dsc)) != 0:
                    raise SystemExit("bench.py: ruyb200_mul_async failed: " + lib().ruyb200_last_error().decode())
            ctx.sync()
            kernel = ctx.counters()["last_kernel"]
            checked = verify_case(case, case.dst_view(sets[-1][0].cpu().numpy()))
            launches0 = ctx.counters()["launches"]
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for dsc in descs:
                    fn(ctx._h, C.byref(dsc))
            launches = (ctx.counters()["launches"] - launches0) / copies
            rounds = max(3, min(args.steps, int(2e-3 / (copies * 5e-6)) + 1))
            graph.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(rounds):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
            ms = e0.elapsed_time(e1) / (rounds * copies)
            # end to end with host operands through the synchronous call
            hdst = case.new_dst()
            hl, hr, hp, hd, hkeep = case.bind(hdst, rounding=Rounding.kReference)
            for _ in range(3):    # the first call packs and caches the weights; the next ones settle the host side
                ruy_b200.mul(hl, hr, hp, ctx, hd)
            per_call = []
            for _ in range(9):
                t0 = time.perf_counter()
                ruy_b200.mul(hl, hr, hp, ctx, hd)
                per_call.append(time.perf_counter() - t0)
            e2e_ms = float(np.median(per_call)) * 1e3   # median: single calls right after a large upload ran 10-50x long
            gops = case.ops / (ms * 1e-3) / 1e9
            gbs = nbytes / (ms * 1e-3) / 1e9
            is_float = case.accum == "float32"
            hbm_time = nbytes / (peaks["hbm_gbs"] * 1e9)
            math_peak = 75e12 if is_float else 2.0 * peaks["bf16_tflops"] * 1e12
            math_time = case.ops / math_peak
            bound = "hbm" if hbm_time >= math_time else "tensor"
            line = {"metric": "mul_time_us", "value": ms * 1e3, "unit": "us", "n_gpus": 1, "steps": rounds * copies, "warmup": copies,
                    "ms_per_step": ms, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
                    "dtype": "f32" if is_float else "int8", "data": "synthetic",
                    "config": {"workload": case.name, "rows": case.rows, "depth": case.depth, "cols": case.cols,
                               "l2": f"activations and destination rotate over {copies} copies ({copies * nbytes >> 20} MiB); "
                                     f"{rounds} graph replays of one pass between one event pair"},
                    "kernel": kernel, "gops": gops, "gpu_launches": launches, "checked": checked,
                    "e2e": {"value": e2e_ms * 1e3, "unit": "us", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None},
                    "roofline": {"bound": bound, "achieved": gbs if bound == "hbm" else gops / 1e3,
                                 "peak": peaks["hbm_gbs"] if bound == "hbm" else math_peak / 1e12,
                                 "unit": "GB/s" if bound == "hbm" else "TFLOP/s",
                                 "frac": (gbs / peaks["hbm_gbs"]) if bound == "hbm" else (gops / 1e3) / (math_peak / 1e12),
                                 "traffic": None,
                                 "peak_source": "measured hbm_gbs" if bound == "hbm" else
                                 ("nominal fp32 FFMA 75 TFLOP/s" if is_float else "2 x measured bf16_tflops")}}
            if ref_ctx is not None and not args.no_cpu_baseline:
                cb = case.bind(case.new_dst())
                cdesc = make_desc(cb[0], cb[1], cb[2], cb[3])
                secs = ref.ruy_ref_time_mul(ref_ctx, C.byref(cdesc), 2, 0.2)
                line["cpu_baseline"] = {"value": secs * 1e6, "unit": "us", "cores": cores, "physical_cores": host["physical_cores"],
                                        "cpu_model": host["cpu_model"], "kind": "reference",
                                        "sample": "the same mul, ruy::Mul on the widest host SIMD path, all host threads, hot cache"}
            print(json.dumps(line), flush=True)
            del graph, sets, descs
            torch.cuda.empty_cache()
    if ref_ctx is not None:
        ref.ruy_ref_ctx_destroy(ref_ctx)
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3_i8", choices=["c3_i8", "c3_i32", "c2", "c0", "c1", "c4", "small", "narrow"])
    ap.add_argument("--muls", type=int, default=16384, help="number of muls of workload c2")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-c2", action="store_true", help="leave the small-mul sub-record out of the default line")
    ap.add_argument("--no-sustained", action="store_true", help="skip the one-second back-to-back measurement")
    ap.add_argument("--only", default="", help="workloads c0/c1/c4/small: run only the cases whose name contains this text")
    ap.add_argument("--gather", default="mirror", choices=["mirror", "nccl"],
                    help="N>1: how the column-sharded destination is gathered (epilogue peer stores, or an NCCL all-gather)")
    ap.add_argument("--cols", type=int, default=8192,
                    help="activation columns (8192 is the benchmark configuration; smaller values are for profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "c2":
        run_c2_arm(args)
    elif args.workload in ("c0", "c1", "c4", "small", "narrow"):
        run_small_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
