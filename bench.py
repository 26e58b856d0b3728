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
import subprocess
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

def run_gpu_arm(args):
    import torch
    import ruy_b200
    from ruy_b200 import cases
    from ruy_b200.api import Rounding

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the GPU arm has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    use_dist = world > 1
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

    stream = torch.cuda.Stream(device=dev)
    ctx = ruy_b200.Context(local, stream=stream.cuda_stream)
    mirrored = use_dist and args.gather == "mirror"
    peer_full = flags = None
    if mirrored:
        from ruy_b200 import peer
        peer_full = peer.PeerBuffer(cols_total * case.rows * esz, dev)
        flags = peer.StepFlags(dev)
    with torch.cuda.stream(stream):
        # the gathered destination (col-major: a column shard is one contiguous range); each rank
        # computes straight into its own slice of it
        if mirrored:
            full = peer_full.tensor.view(tdtype)
        else:
            full = torch.zeros(cols_total * case.rows, dtype=tdtype, device=dev)
        mine = full[rank * shard * case.rows:(rank + 1) * shard * case.rows]
        lhs, rhs, p, d, keep = case.bind(mine, device=dev, rounding=Rounding.kReference)
        flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
        ruy_b200.mul(lhs, rhs, p, ctx, d)  # packs the weights into the context's device cache
        shard_bytes = shard * case.rows * esz
        mirror_ptrs = [q + rank * shard_bytes for r_, q in enumerate(peer_full.ptrs) if r_ != rank] if mirrored else []
        step_no = [0]

        def compute():
            if mirrored:
                # the epilogue stores each tile here and in every peer's buffer: the gather rides along with the math
                peer.mul_async_mirrored(lhs, rhs, p, ctx, d, mirror_ptrs)
            else:
                ruy_b200.mul_async(lhs, rhs, p, ctx, d)

        def finish():
            if mirrored:
                step_no[0] += 1
                flags.signal_and_wait(ctx, step_no[0])      # every peer's tiles have landed in this rank's buffer
            elif use_dist:
                dist.all_gather_into_tensor(full, mine)

        def step():
            compute()
            finish()

        sampler = ClockSampler(local)
        sampler.start()
        for _ in range(max(args.warmup, 3)):
            flush.fill_(1)
            step()
        stream.synchronize()

        # correctness spot check (cheap): a sampled sub-block against 64-bit numpy dot products
        out = case.dst_view(mine.cpu().numpy())
        rs = np.arange(0, case.rows, 509)
        cs = np.arange(0, shard, 211)
        L = case.lhs.reshape(case.rows, case.depth).astype(np.int64)[rs]
        R = case.rhs.reshape(shard, case.depth).astype(np.int64)[cs]
        acc = L @ R.T
        if dst_name == "int8":
            acc = acc + case.bias.astype(np.int64)[rs][:, None]
            m, e = case.mfp.astype(np.int64)[rs][:, None], case.mexp.astype(np.int64)[rs][:, None]
            acc = np.clip(((acc * m + (1 << (30 - e))) >> (31 - e)) + case.dst_zp, -128, 127)
        if not np.array_equal(out[np.ix_(rs, cs)].astype(np.int64), acc):
            raise SystemExit("bench.py: GPU result does not match the reference arithmetic; refusing to report")
        if use_dist:
            # the gathered part: a sample of the next rank's columns must have arrived here
            nb = (rank + 1) % world
            nb_case = cases.config3(dst=dst_name, col_begin=nb * shard, col_count=shard)
            nb_out = nb_case.dst_view(full[nb * shard * case.rows:(nb + 1) * shard * case.rows].cpu().numpy())
            accn = L @ nb_case.rhs.reshape(shard, case.depth).astype(np.int64)[cs].T
            if dst_name == "int8":
                accn = accn + case.bias.astype(np.int64)[rs][:, None]
                accn = np.clip(((accn * m + (1 << (30 - e))) >> (31 - e)) + case.dst_zp, -128, 127)
            if not np.array_equal(nb_out[np.ix_(rs, cs)].astype(np.int64), accn):
                raise SystemExit("bench.py: the gathered destination is wrong; refusing to report")

        launches0 = ctx.counters()["launches"]
        if use_dist:
            dist.barrier()
        torch.cuda.synchronize()
        sampler.mark_begin()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        mids = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        wall0 = time.perf_counter()
        for i in range(args.steps):
            flush.fill_(i & 0xFF)          # evict the operands from L2 (not timed)
            starts[i].record(stream)
            compute()
            mids[i].record(stream)
            finish()
            stops[i].record(stream)
        stream.synchronize()
        if use_dist:
            dist.barrier()
        torch.cuda.synchronize()
        wall = time.perf_counter() - wall0
        sampler.mark_end()
        clocks = sampler.stop()
        launches = ctx.counters()["launches"] - launches0
        step_ms = [s.elapsed_time(e) for s, e in zip(starts, stops)]
        kern_ms = [s.elapsed_time(e) for s, e in zip(starts, mids)]
        total_ms = float(np.sum(step_ms))
        kernel_ms = float(np.mean(kern_ms))
        if use_dist:
            t = torch.tensor([total_ms, kernel_ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            total_ms, kernel_ms = float(t[0]), float(t[1])
        ms_per_step = total_ms / args.steps
        total_ops = 2.0 * case.rows * case.depth * cols_total
        value = total_ops / (ms_per_step * 1e-3) / 1e12

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
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            ruy_b200.mul(hl, hr, hp, ctx, hd)
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
        if not np.array_equal(case.dst_view(pinned_dst.numpy())[np.ix_(rs, cs)].astype(np.int64), acc):
            raise SystemExit("bench.py: end-to-end result mismatch")

    peaks = measured_peaks()
    # tcgen05 kind::i8 issues twice the multiply-adds per clock of kind::f16: the int8 dense peak is
    # taken as 2 x the measured dense bf16 throughput (the burst figure: the kernel is timed alone).
    peak_tops = 2.0 * peaks["bf16_tflops"]
    shard_ops = 2.0 * case.rows * case.depth * shard
    achieved = shard_ops / (kernel_ms * 1e-3) / 1e12
    # DRAM bytes per launch of this kernel from the ncu launch list (profiles/tc_i8_kernel_c3_launch_list.md):
    # 50.5 MB read + 2.8 MB written for the full 8192-column int8 workload on one GPU; not measured elsewhere.
    traffic = 53.3e6 if (world == 1 and cols_total == 8192 and dst_name == "int8") else None
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak_tops, "unit": "TFLOP/s",
                "frac": achieved / peak_tops, "traffic": traffic, "kernel": "tc_i8_kernel",
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
                        ("epilogue stores into peers' memory over NVLink + flag exchange" if mirrored else "an NCCL all-gather"))
                       if use_dist else ""),
                   "l2": f"flushed between steps ({L2_FLUSH_BYTES >> 20} MiB fill, untimed)"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "ms_per_step": e2e_s * 1e3},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": roofline,
        "wall_s": wall,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        arm = CpuArm(args.workload)
        secs = arm.seconds(windows=4, min_secs=0.5 if arm.kind == "reference" else 0.0)
        line["cpu_baseline"] = {"value": arm.tops(secs), "unit": UNIT, "cores": arm.cores, "kind": arm.kind,
                                "sample": arm.describe()}
        arm.close()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if mirrored:
        ctx.sync()
        flags.close()
        peer_full.close()
    ctx.close()
    if use_dist:
        dist.destroy_process_group()


def run_c2_arm(args):
    """Batched small muls (config 2): 16384 independent int8 muls with dims drawn from {16..128}, weights in the
    prepacked cache, one plan replayed per step with a single persistent launch.  With N ranks the mul index
    range is split evenly (no collective: the destinations stay where their consumers are)."""
    import torch
    import ruy_b200
    from ruy_b200 import _abi, cases
    from ruy_b200.api import CachePolicy, Layout, Matrix, MulParams, Order, Rounding

    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    from ruy_b200.sharding import mul_range
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
        # parity spot check against the CPU oracle on a few muls of this rank
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import util
        host_dst = dst_buf.cpu().numpy()
        for i in list(range(0, len(mine), max(1, len(mine) // 8)))[:8]:
            c = mine[i]
            got = c.dst_view(host_dst[dst_off[i]:dst_off[i] + c.dst_storage_elems()])
            if not np.array_equal(got, util.run_oracle(c, Rounding.kReference)):
                raise SystemExit(f"bench.py: mul {first + i} does not match the oracle; refusing to report")
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
        ms = float(np.sum([a.elapsed_time(b) for a, b in zip(starts, stops)])) / args.steps
        if use_dist:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
            tb = torch.tensor([float(nbytes), float(ops)], dtype=torch.float64, device=dev)
            dist.all_reduce(tb)
            total_bytes, total_ops = float(tb[0]), float(tb[1])
        else:
            total_bytes, total_ops = float(nbytes), float(ops)
    peaks = measured_peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    line = {
        "metric": "small_mul_muls_per_s", "value": n_total / (ms * 1e-3), "unit": "muls/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "c2", "muls": n_total, "dims": list(cases.CONFIG2_DIMS),
                   "sharding": f"{world} shard(s) by mul index", "l2": f"flushed between steps ({L2_FLUSH_BYTES >> 20} MiB fill, untimed)",
                   "plan_build_s": plan_build_s},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                     # DRAM bytes per launch from the ncu capture of the full 16384-mul plan on one GPU
                     # (profiles/batch_i8_kernel_c2_full_set.md: 152.1 MB read + 40.3 MB written); not measured elsewhere
                     "traffic": 192.4e6 if (world == 1 and n_total == 16384) else None,
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
            cores = os.cpu_count() or 1
            secs = ref.ruy_ref_time_batch(host_descs, len(sample), cores, oracle.host_simd_path(), 5)
            line["cpu_baseline"] = {"value": len(sample) / secs, "unit": "muls/s", "cores": cores, "kind": "reference",
                                    "sample": f"first {len(sample)} of {n_total} muls; {cores} host threads, one ruy::Context each, "
                                              "LHS in ruy's prepacked cache"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    plan.close()
    ctx.close()
    if use_dist:
        dist.destroy_process_group()


def run_small_arm(args):
    """The remaining benchmark configurations, one JSON line each (single GPU, device-resident operands, the
    stream-ordered entry point timed with CUDA events; L2 flushed between calls): config 0 (256x512x128 int8),
    config 1 (the five fp32 shapes) and config 4 (the uint8 pointwise-conv layers at batch 1 and 64).  Every
    line carries the same mul timed through ruy's own CPU path on all host cores."""
    import torch
    import ruy_b200
    from ruy_b200 import cases
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
    ref = oracle.reference()
    cores = os.cpu_count() or 1
    ref_ctx = ref.ruy_ref_ctx_create(oracle.host_simd_path(), cores) if ref is not None else None
    torch_dt = {"int8": torch.int8, "uint8": torch.uint8, "int32": torch.int32, "float32": torch.float32}
    with torch.cuda.stream(stream):
        flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
        for case in todo:
            dst = torch.zeros(case.dst_storage_elems(), dtype=torch_dt[case.dst_dtype], device=dev)
            lhs, rhs, p, d, keep = case.bind(dst, device=dev, rounding=Rounding.kReference)
            ruy_b200.mul(lhs, rhs, p, ctx, d)
            kernel = ctx.counters()["last_kernel"]
            for _ in range(3):
                flush.fill_(1)
                ruy_b200.mul_async(lhs, rhs, p, ctx, d)
            stream.synchronize()
            steps = min(args.steps, 50)
            starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
            stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
            launches0 = ctx.counters()["launches"]
            for i in range(steps):
                flush.fill_(i & 0xFF)
                starts[i].record(stream)
                ruy_b200.mul_async(lhs, rhs, p, ctx, d)
                stops[i].record(stream)
            stream.synchronize()
            launches = (ctx.counters()["launches"] - launches0) / steps
            ms = float(np.median([a.elapsed_time(b) for a, b in zip(starts, stops)]))
            # end to end with host operands through the synchronous call
            hdst = case.new_dst()
            hl, hr, hp, hd, hkeep = case.bind(hdst, rounding=Rounding.kReference)
            ruy_b200.mul(hl, hr, hp, ctx, hd)
            t0 = time.perf_counter()
            reps = 5
            for _ in range(reps):
                ruy_b200.mul(hl, hr, hp, ctx, hd)
            e2e_ms = (time.perf_counter() - t0) / reps * 1e3
            nbytes = case.algorithmic_bytes()
            gops = case.ops / (ms * 1e-3) / 1e9
            gbs = nbytes / (ms * 1e-3) / 1e9
            is_float = case.accum == "float32"
            hbm_time = nbytes / (peaks["hbm_gbs"] * 1e9)
            math_peak = 75e12 if is_float else 2.0 * peaks["bf16_tflops"] * 1e12
            math_time = case.ops / math_peak
            bound = "hbm" if hbm_time >= math_time else "tensor"
            line = {"metric": "mul_time_us", "value": ms * 1e3, "unit": "us", "n_gpus": 1, "steps": steps, "warmup": 3,
                    "ms_per_step": ms, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
                    "dtype": "f32" if is_float else "int8", "data": "synthetic",
                    "config": {"workload": case.name, "rows": case.rows, "depth": case.depth, "cols": case.cols,
                               "l2": "flushed between steps"},
                    "kernel": kernel, "gops": gops, "gpu_launches": launches,
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
                line["cpu_baseline"] = {"value": secs * 1e6, "unit": "us", "cores": cores, "kind": "reference",
                                        "sample": "the same mul, ruy::Mul on the widest host SIMD path, all host threads, hot cache"}
            print(json.dumps(line), flush=True)
    if ref_ctx is not None:
        ref.ruy_ref_ctx_destroy(ref_ctx)
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3_i8", choices=["c3_i8", "c3_i32", "c2", "c0", "c1", "c4", "small"])
    ap.add_argument("--muls", type=int, default=16384, help="number of muls of workload c2")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gather", default="mirror", choices=["mirror", "nccl"],
                    help="N>1: how the column-sharded destination is gathered (epilogue peer stores, or an NCCL all-gather)")
    ap.add_argument("--cols", type=int, default=8192,
                    help="activation columns (8192 is the benchmark configuration; smaller values are for profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "c2":
        run_c2_arm(args)
    elif args.workload in ("c0", "c1", "c4", "small"):
        run_small_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
