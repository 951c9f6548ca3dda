#!/usr/bin/env python
"""Benchmark of the elementwise / reduce hot path: effective HBM GB/s per op.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-per-op]

Headline workload (benchmark configuration 2): the fused chain z = sigmoid(x) * y + exp(-abs(x)) over
2^28 fp32 elements per GPU (x ~ N(0,1) seed 0, y ~ N(0,1) seed 1), one step = one pass = one
launch of plast_b200_chain_forward. Algorithmic bytes per element: 12 (read x, y; write z).
The 3 GiB working set is far larger than L2, so no flush is needed between steps.

For N > 1 (torchrun, one rank per GPU) every rank runs its own 2^28-element shard (weak
scaling, no data-path collective: an elementwise op shards along its outermost dim); time is the
max over ranks of the CUDA-event time; value is the whole-job GB/s.

`--impl reference` times the reference's own CPU kernels (oracle/_ref, else the oracle port) on
the host cores for the same chain, on a bounded sample of the workload.

One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHARDED_TABLE_LIMIT_S = 240  # wall-clock limit of the multi-GPU per-op table (seconds)
N_ELEMS = 1 << 28
BYTES_PER_ELEM = 12
METRIC = "effective_hbm_gbps"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0

CHAIN_STEPS = [("neg", 0, 0, 0.0), ("exp", 2, 0, 0.0), ("add_scalar", 3, 0, 1.0),
               ("rdiv_scalar", 4, 0, 1.0), ("mul", 5, 1, 0.0), ("abs", 0, 0, 0.0),
               ("neg", 7, 0, 0.0), ("exp", 8, 0, 0.0), ("add", 6, 9, 0.0)]


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ---- reference / oracle CPU arm -------------------------------------------------------------------
def cpu_chain_baseline(n_sample: int, reps: int):
    """Times the 9-op chain through the reference's CPU entry points (kind 'reference') or the
    oracle port (kind 'port') on n_sample elements; returns (GB/s by the 12 B/el count, info)."""
    sys.path.insert(0, str(ROOT / "tests"))
    import plast_b200 as pb
    from harness import CpuBackend, have_ref, build_oracle
    if have_ref():
        be, kind = CpuBackend("ref"), "reference"
    else:
        build_oracle()
        be, kind = CpuBackend("oracle"), "port"
    cores = os.cpu_count() or 1
    os.environ.setdefault("OMP_NUM_THREADS", str(cores))
    rs = np.random.RandomState(0)
    x = be.tensor(rs.randn(n_sample).astype(np.float32))
    y = be.tensor(np.random.RandomState(1).randn(n_sample).astype(np.float32))
    one = be.tensor(np.float32(1.0).reshape(()))
    t = [be.empty((n_sample,)) for _ in range(9)]

    def chain():
        be.forward("neg", [x], t[0]); be.forward("exp", [t[0]], t[1]); be.forward("add", [t[1], one], t[2])
        be.forward("div", [one, t[2]], t[3]); be.forward("mul", [t[3], y], t[4]); be.forward("abs", [x], t[5])
        be.forward("neg", [t[5]], t[6]); be.forward("exp", [t[6]], t[7]); be.forward("add", [t[4], t[7]], t[8])

    chain()
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        chain()
        times.append(time.perf_counter() - t0)
    best = min(times)
    gbs = BYTES_PER_ELEM * n_sample / best / 1e9
    info = {"value": gbs, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": f"9-op chain (neg,exp,+1,1/.,mul,abs,neg,exp,add) on 2^{int(np.log2(n_sample))} "
                      f"of the 2^28 elements, best of {reps}, {best * 1e3:.1f} ms; contiguous "
                      "elementwise kernels of the reference are single-threaded by construction"}
    return gbs, info, float(np.mean(times))


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_sample = 1 << 24
    # K + W steps, each one pass of the chain over the sample
    sys.path.insert(0, str(ROOT / "tests"))
    gbs, info, _ = cpu_chain_baseline(n_sample, max(1, args.steps + args.warmup))
    ms = BYTES_PER_ELEM * n_sample / (gbs * 1e9) * 1e3
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config 2: fused chain z = sigmoid(x)*y + exp(-abs(x)), fp32, "
                               f"bounded sample of 2^24 of 2^28 elements per step",
                   "l2": "n/a (host)"},
        "cpu_baseline": info,
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---- clocks -----------------------------------------------------------------------------------------
class ClockSampler:
    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.reasons = set()
        self._stop = threading.Event()
        self._th = None
        self.max_mhz = None

    def _init_nvml(self) -> bool:
        """NVML handle for the sampled GPU, set up BEFORE the timed region starts."""
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = None
            try:
                import torch
                uuid = "GPU-" + str(torch.cuda.get_device_properties(self.index).uuid)
                h = nv.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                h = None
            if h is None:
                h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            self._nv, self._h = nv, h
            self._bits = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
                          "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                          "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
                          "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
            return True
        except Exception:
            self._nv = None
            return False

    def _run_nvml(self) -> bool:
        """NVML queries take well under a millisecond, so even a short timed region is sampled."""
        nv = getattr(self, "_nv", None)
        if nv is None:
            return False
        while True:
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for n, b in self._bits.items():
                    if r & b:
                        self.reasons.add(n)
            except Exception:
                pass
            if self._stop.wait(0.002):
                break
        return True

    def _run(self):
        if self._run_nvml():
            return
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                f = [s.strip() for s in out.strip().split(",")]
                self.samples.append(float(f[0]))
                self.max_mhz = float(f[1])
                for n, v in zip(names, f[2:6]):
                    if v.lower().startswith("active"):
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(0.1)

    def start(self):
        self._init_nvml()
        self._th = threading.Thread(target=self._run, daemon=True)
        self._th.start()

    def stop(self):
        self._stop.set()
        if self._th:
            self._th.join(timeout=10)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ---- our arm ----------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    import plast_b200 as pb

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ["NCCL_DEBUG"] = "WARN"  # keep NCCL's version banner off stdout (one JSON line)
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # launches go to torch's current stream so torch events bracket them
    pb.lib.plast_b200_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))

    n = args.elems
    # configuration 2 inputs; rank r draws seeds (2r, 2r+1) so shards differ
    x_h = torch.from_numpy(np.random.RandomState(2 * rank).randn(n).astype(np.float32)).pin_memory()
    y_h = torch.from_numpy(np.random.RandomState(2 * rank + 1).randn(n).astype(np.float32)).pin_memory()
    z_h = torch.empty(n, dtype=torch.float32).pin_memory()
    x_d = torch.empty(n, dtype=torch.float32, device=dev)
    y_d = torch.empty(n, dtype=torch.float32, device=dev)
    z_d = torch.empty(n, dtype=torch.float32, device=dev)
    x_d.copy_(x_h); y_d.copy_(y_h)

    def wrap(t):
        """plast Tensor struct over a torch allocation (no copy)."""
        return pb.Tensor.wrap_pointer(t.data_ptr(), list(t.shape), owner=t)

    X, Y, Z = wrap(x_d), wrap(y_d), wrap(z_d)

    def step():
        pb.chain_forward([X, Y], Z, CHAIN_STEPS, check=False)

    step(); pb.check_error()
    torch.cuda.synchronize()
    # parity spot-check of the timed kernel against the oracle on a slice (outside the timed region)
    if rank == 0:
        sys.path.insert(0, str(ROOT / "tests"))
        from harness import OracleRecipes
        sl = slice(0, 1 << 16)
        xs, ys = x_h[sl].numpy(), y_h[sl].numpy()
        want = OracleRecipes().chain(xs, ys).astype(np.float64)
        got = z_d[sl].cpu().numpy().astype(np.float64)
        x64, y64 = xs.astype(np.float64), ys.astype(np.float64)
        terms = np.abs(y64) / (1 + np.exp(-x64)) + np.exp(-np.abs(x64))  # z = t + e2 may cancel
        assert (np.abs(got - want) <= 4 * 2.0 ** -23 * terms).all(), "bench: fused chain disagrees with the oracle"

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    l0 = pb.lib.plast_b200_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    launches = int(pb.lib.plast_b200_launch_count() - l0)
    ms_total = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total_max = float(t.item())
    ms_per_step = ms_total_max / args.steps
    total_bytes = BYTES_PER_ELEM * n * world
    value = total_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- end to end: host buffers in, host buffer out, copies inside the timed region ----------
    # The library's host-buffer entry point: pinned host arrays in, pinned host array out; chunks
    # are copied in, computed and copied out on three streams at once.
    host_in = [(x_h.data_ptr(), n), (y_h.data_ptr(), n)]
    host_out = (z_h.data_ptr(), n)

    def e2e_step():
        pb.chain_forward_host(host_in, host_out, CHAIN_STEPS, check=False)

    e2e_steps = min(args.steps, 10)
    z_h.zero_()
    e2e_step(); pb.check_error(); barrier()
    if rank == 0:   # the host result of the pipelined call equals the device-resident one
        assert torch.equal(z_h[: 1 << 20], z_d[: 1 << 20].cpu()) and torch.equal(z_h[-(1 << 20):], z_d[-(1 << 20):].cpu()), \
            "bench: host-buffer chain disagrees with the device-resident chain"
    ev0.record()
    for _ in range(e2e_steps):
        e2e_step()
    ev1.record()
    barrier()
    t = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / e2e_steps
    e2e = {"value": total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": 8 * n, "d2h_bytes_per_step": 4 * n, "steps": e2e_steps,
           "call": "plast_b200_chain_forward_host (pinned host buffers; 32 MiB chunks; copy-in, kernel and "
                   "copy-out of successive chunks overlap)"}

    peak, peak_kind = measured_peak()
    achieved = BYTES_PER_ELEM * n / (ms_total / args.steps * 1e-3) / 1e9  # this rank's kernel
    roofline = {"bound": "hbm", "kernel": "ew_kernel<SigmoidMulAddExpNegAbs, vec4, 1-D>",
                "achieved": achieved, "peak": peak, "peak_source": f"of {peak_kind}", "unit": UNIT,
                "frac": achieved / peak, "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
                "traffic": None, "algorithmic_bytes_per_launch": BYTES_PER_ELEM * n}
    # per-launch DRAM traffic from the committed ncu summary (measured at 2^26 elements, scaled)
    prof = ROOT / "profiles" / "ew_kernel_chain_config2.md"
    if prof.exists() and n == N_ELEMS:
        import re
        m = re.search(r"^dram_bytes_per_launch\s*=\s*(\d+)", prof.read_text(), flags=re.M)
        if m:
            roofline["traffic"] = int(m.group(1))
            roofline["traffic_source"] = "ncu dram__bytes_read+write on 2^26 elements x4, profiles/ew_kernel_chain_config2.md"

    per_op = None
    if rank == 0 and world == 1 and not args.no_per_op:
        from plast_b200.opbench import per_op_table
        del x_h, y_h, z_h
        per_op = per_op_table(torch, pb, dev, peak, reps=args.op_reps,
                              configs=tuple(int(c) for c in args.configs.split(",")), chain_elems=args.elems)

    def headline(extra):
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "config 2: fused chain z = sigmoid(x)*y + exp(-abs(x)) on 2^28 fp32 "
                                   "elements per GPU, x,y ~ N(0,1) (numpy RandomState seeds 0,1)",
                       "algorithmic_bytes_per_element": BYTES_PER_ELEM, "elements_per_gpu": n,
                       "is_baseline_size": n == N_ELEMS,
                       "l2": "working set 3 GiB per GPU > 126 MB L2; no flush needed",
                       "sharding": "elements split across ranks, no collective"},
            "elements_per_s": n * world / (ms_per_step * 1e-3),
            "roofline": roofline, "cpu_baseline": cpu_info, "e2e": e2e, "gpu_launches": launches,
            "clocks": clocks,
        }
        if per_op is not None:
            line["per_op"] = per_op
        line.update(extra)
        return line

    cpu_info = None
    if rank == 0 and world == 1:
        _, cpu_info, _ = cpu_chain_baseline(1 << 25, 40)   # about 12 s of CPU work

    sharded = None
    if world > 1 and not args.no_per_op:
        # Strong scaling of the fixed config 3 / 4 / 5 tensors split across the ranks (local kernel
        # + exchange); every rank takes part. The headline above is already measured: if this
        # extra table does not come back within its time limit (a collective that never completes),
        # rank 0 still prints the JSON line, without the table, and every rank leaves.
        import threading
        from plast_b200.dist import sharded_reduction_table
        del x_h, y_h, z_h
        printed = threading.Lock()

        def give_up():
            if rank == 0 and printed.acquire(blocking=False):
                print(json.dumps(headline({"sharded_reductions_error": "timed out after %d s" % SHARDED_TABLE_LIMIT_S})),
                      flush=True)
            os._exit(0)

        watchdog = threading.Timer(SHARDED_TABLE_LIMIT_S, give_up)
        watchdog.daemon = True
        watchdog.start()
        try:
            sharded = sharded_reduction_table(torch, dist, pb, dev, peak, reps=args.op_reps)
        except Exception as exc:  # the table is an extra: never lose the headline to it
            sharded = [{"op": "sharded_table_failed", "error": str(exc)[:200]}]
        watchdog.cancel()
        if rank == 0 and not printed.acquire(blocking=False):
            return  # the watchdog is printing

    if rank == 0:
        print(json.dumps(headline({"sharded_reductions": sharded} if sharded is not None else {})), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_per_op_only(args):
    import torch
    import plast_b200 as pb
    from plast_b200.opbench import per_op_table
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    pb.lib.plast_b200_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))
    peak, kind = measured_peak()
    cfgs = tuple(int(c) for c in args.configs.split(","))
    rows = per_op_table(torch, pb, dev, peak, reps=args.op_reps, configs=cfgs, chain_elems=args.elems)
    print(json.dumps({"per_op": rows, "peak_gbs": peak, "peak_source": f"of {kind}"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--elems", type=int, default=N_ELEMS,
                    help="elements per GPU (default 2^28, the benchmark size; smaller only for profiler captures)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-per-op", action="store_true", help="skip the per-op table (configs 1-5 and the optimiser steps)")
    ap.add_argument("--op-reps", type=int, default=10)
    ap.add_argument("--per-op-only", action="store_true",
                    help="only the per-op table (1 GPU); with --op-reps 0 every op is launched 3 times and "
                         "not timed, which is the command the profiler captures use")
    ap.add_argument("--configs", default="1,2,3,4,5,6", help="configs of the per-op table (6 = optimiser steps)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.per_op_only:
        run_per_op_only(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
