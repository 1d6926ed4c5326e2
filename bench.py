#!/usr/bin/env python
"""Benchmark of the epsilon self-join hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3] [--impl reference]

A *step* is one pass of the hot path over the workload: row norms + the join of this rank's
query band against all candidates (the interval the reference calls "Total Kernel Elapsed
time", source/findPairs.cuh:728-748 of the reference).  The metric is the reference's:
TFLOPS = 2 * N * N * D / seconds / 1e12 over the un-padded N and D.

One JSON line is printed by rank 0:
  value      device-timed throughput with the dataset already resident in HBM
  e2e        the same metric through the public API with HOST buffers: pinned host -> device copy
             of the dataset (plus the NCCL broadcast at N > 1), norms, join, sort, and the
             device -> host copy of the pair list, every step
  roofline   the join kernel against the measured tensor-core peak
  cpu_baseline  an OpenMP FP64 brute-force self-join on a bounded sample, on the host cores

`--impl reference` times the CPU baseline alone (the reference has no CPU implementation of the
join and its GPU implementation is what this library replaces; the FP64 OpenMP brute force is
the CPU arm its task definition names).

Multi-GPU: launched by torchrun with one rank per GPU; total work is fixed (strong scaling):
rank r joins query rows [r*B, (r+1)*B) against all N candidates after one NCCL broadcast of the
FP16 matrix.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from fasted_b200.workloads import SEED, WORKLOADS, fill_device, host_sample as make_host_sample  # noqa: E402

PUBLISHED_A100_TFLOPS = {"c3": 153.64}  # mean of the reference's three 1,000,000 x 4096 trials (A100 PCIe)
NOMINAL_FP16_TFLOPS = 2250.0


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(burst=p.get("bf16_tflops"), sustained=p.get("bf16_tflops_sustained"), hbm=p.get("hbm_gbs"),
                    source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU every 200 ms while running."""

    def __init__(self, index: int):
        self.index, self.samples, self.reasons = index, [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake_slowdown",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.2)

    def start(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._thread:
            self._thread.join()
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def cpu_fp64_sample(pts: np.ndarray, d: int, eps: float, q_rows: int) -> dict:
    """Times the OpenMP FP64 brute force (the checker's, used here only as the reported CPU baseline)."""
    import oracle
    c_rows = pts.shape[0]
    t0 = time.perf_counter()
    _, _, found = oracle.join_fp64(pts, eps, d=d, q_begin=0, q_end=q_rows, capacity=1)
    dt = time.perf_counter() - t0
    return {"value": 2.0 * q_rows * c_rows * d / dt / 1e12, "unit": "TFLOPS", "cores": oracle.num_threads(),
            "kind": "port", "seconds": dt,
            "sample": f"{q_rows} query rows x {c_rows} candidate rows x {d} dims, FP64 direct form, OpenMP"}


def size_cpu_sample(wl: dict, budget_flop: float) -> tuple[int, int]:
    c_rows = min(wl["n"], 32768)
    q_rows = int(max(16, min(c_rows, budget_flop / (2.0 * c_rows * wl["d"]))))
    return q_rows, c_rows


def run_reference_arm(args, wl: dict, name: str) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun sets OMP_NUM_THREADS=1 for its children; this arm is the only rank that works and is
    # meant to use all host threads (the OpenMP runtime reads the variable when it is first loaded).
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 and os.environ.get("OMP_NUM_THREADS") == "1":
        os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    import oracle
    cores = oracle.num_threads()
    q_rows, c_rows = size_cpu_sample(wl, budget_flop=1e12 * cores / 16)
    pts = make_host_sample(wl, c_rows)
    eps = wl["eps"] if wl["eps"] else 1.0
    for _ in range(args.warmup):
        cpu_fp64_sample(pts, wl["d"], eps, max(16, q_rows // 8))
    t0 = time.perf_counter()
    last = None
    for _ in range(args.steps):
        last = cpu_fp64_sample(pts, wl["d"], eps, q_rows)
    dt = (time.perf_counter() - t0) / args.steps
    value = 2.0 * q_rows * c_rows * wl["d"] / dt / 1e12
    line = {
        "impl": "reference", "metric": "self_join_tflops", "value": value, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": f"{name}: self-join {wl['n']} x {wl['d']} {wl['dist']}; CPU arm on a bounded sample",
                   "n": wl["n"], "d": wl["d"], "epsilon": eps},
        "cpu_baseline": {"value": value, "unit": "TFLOPS", "cores": cores, "kind": "port", "sample": last["sample"]},
        "e2e": {"value": value, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def reference_gpu_leg(sj_cls, dev_pts, wl: dict, eps: float, rows: int) -> dict:
    """The reference's own kernels on this GPU beside this library, on the SAME buffer: the first `rows`
    points of the workload.  oracle/_ref/ref_join is the reference's findPairs.cuh compiled unmodified for
    sm_100 behind a file-in / file-out harness (test infrastructure; built where the reference checkout is
    mounted).  Both figures use the reference's timer: row norms + join kernel, 2*n*n*d flop.  Outside
    every timed region of the benchmark; never part of `value`."""
    import re
    import subprocess
    import tempfile
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_join")
    d = wl["d"]
    m = min(rows, wl["n"])
    if not os.path.exists(exe):
        return {"unavailable": "oracle/_ref/ref_join is not built (it is compiled from the reference checkout)"}
    with sj_cls(dev_pts.device.index or 0) as sj2:
        sj2.set_points_device(dev_pts.data_ptr(), m, d, dev_pts.shape[1], keepalive=dev_pts)
        for _ in range(2):
            st = sj2.join(eps, capacity=max(m * 256, 1 << 20))
        ours = sj2.pairs()
        ours_tflops = 2.0 * m * m * d / (st.kernel_ms * 1e-3) / 1e12
    if st.pairs_found > 20_000_000 or st.pairs_found != st.pairs_stored:
        return {"unavailable": f"{st.pairs_found} pairs on the first {m} points: too many for the reference's "
                               "one-flush-per-pair text output"}
    with tempfile.TemporaryDirectory() as tmp:
        pin = os.path.join(tmp, "p.bin")
        with open(pin, "wb") as f:
            f.write(np.array([m, d], dtype=np.int64).tobytes())
            f.write(dev_pts[:m, :d].contiguous().cpu().numpy().view(np.uint16).tobytes())
        prefix = os.path.join(tmp, "out")
        try:
            r = subprocess.run([exe, pin, repr(eps), prefix], capture_output=True, text=True, timeout=900)
        except subprocess.TimeoutExpired:
            return {"unavailable": "ref_join did not finish within 900 s"}
        mm = re.search(r"REF_RESULTS (\S+) (\S+) (\d+) (\d+)", r.stdout)
        if r.returncode != 0 or not mm:
            return {"unavailable": "ref_join failed: " + (r.stdout[-200:] + r.stderr[-200:]).replace("\n", " ")}
        ref_pairs = np.array(re.findall(r"(\d+), (\d+)", open(prefix + ".pairs").read()), dtype=np.int32).reshape(-1, 2)
    return {"n": m, "d": d, "epsilon": eps, "ref_tflops": float(mm.group(2)), "ours_tflops": ours_tflops,
            "speedup": ours_tflops / float(mm.group(2)), "ref_pairs": int(mm.group(3)), "ours_pairs": int(st.pairs_found),
            "same_pairs": bool(np.array_equal(ref_pairs, ours)),
            "what": "the reference's findPairs.cuh (mma.sync, compiled unmodified for sm_100) and this library on the "
                    "same FP16 buffer on this GPU; TFLOPS = 2*n*n*d / (norm kernel + join kernel), full schedule"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--points", type=int, default=0, help="override the number of points")
    ap.add_argument("--dims", type=int, default=0, help="override the dimension")
    ap.add_argument("--eps", type=float, default=0.0, help="override epsilon (default: workload table or tuned)")
    ap.add_argument("--band-tiles", type=int, default=0)
    ap.add_argument("--cta-pair", type=int, default=-1, help="1: CTA-pair (2-SM) join kernel, 0: single-CTA kernel")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the symmetric-mode and accuracy legs")
    ap.add_argument("--no-refgpu", action="store_true", help="skip the reference's own kernels on this GPU")
    ap.add_argument("--e2e-mode", default="stream", choices=["stream", "serial"],
                    help="N = 1: stream = fasted_join_stream (egress pipelined behind the join); serial = fasted_join, "
                         "then fasted_get_pairs (sort and copy after the join, as the reference orders them)")
    ap.add_argument("--join-behind-load", type=int, default=1, choices=[0, 1],
                    help="N > 1, end-to-end leg: 1 = every rank starts joining the first chunks of its own band while "
                         "the matrix is still being uploaded and all-gathered (fasted_join_stream_arriving); 0 = the "
                         "join's first launch waits for the whole load")
    ap.add_argument("--lead-rows", type=int, default=0,
                    help="query rows per rank joined while the matrix arrives (0 = the library's choice)")
    ap.add_argument("--loader-pieces", type=int, default=0,
                    help="N > 1, end-to-end leg: pieces in which a rank's band is uploaded and all-gathered (1 = upload, "
                         "then one all-gather; 0 = 16 up to 4 GPUs, 8 beyond: the rows a rank joins while the matrix "
                         "arrives lie in the first piece of its band, and with more GPUs the load is a larger part of "
                         "the band's work, so the first piece has to be a larger part of the band)")
    ap.add_argument("--no-numa", action="store_true", help="N > 1: do not pin the rank to its GPU's CPU cores")
    ap.add_argument("--no-balance", action="store_true", help="N > 1: keep equal bands (no sizing by measured rate)")
    ap.add_argument("--option", action="append", default=[], help="name=value for fasted_set_option (tuning runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)

    name = args.workload
    wl = dict(WORKLOADS[name])
    if args.points:
        wl["n"], wl["eps"] = args.points, None
    if args.dims:
        wl["d"], wl["eps"] = args.dims, None
    if (args.points or args.dims) and wl["dist"] == "exp_ref":
        wl["dist"] = "exp"
    if args.eps:
        wl["eps"] = args.eps

    if args.impl == "reference":
        run_reference_arm(args, wl, name)
        return

    import torch
    import torch.distributed as dist
    from fasted_b200 import SelfJoin, JOIN_NO_SORT
    from fasted_b200.dist import (GpuBandEngine, SharedChunkTable, SharedPairBuffer, allgather_points, band_bounds,
                                  dealt_self_join, sharded_self_join, upload_and_allgather)
    from fasted_b200.dist import band_rows as equal_band_rows
    from fasted_b200.dist import load_and_join

    def rows_per_band(n_rows: int, ranks: int) -> int:
        # bands that can be cut into --loader-pieces pieces of whole 256-row candidate tiles
        return equal_band_rows(n_rows, ranks, 256 * max(1, args.loader_pieces))

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.loader_pieces <= 0:
        args.loader_pieces = 16 if world <= 4 else 8
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    numa_cores = None
    if world > 1 and not args.no_numa:
        # before any page-locked buffer exists: the rank's host buffers should live next to its GPU
        from fasted_b200.dist import bind_to_gpu_numa_node
        numa_cores = bind_to_gpu_numa_node(local_rank)
    if world > 1:
        # Rank 0's stdout is the one JSON line: NCCL's version banner (NCCL_DEBUG=VERSION prints it to
        # stdout) is switched off, anything else NCCL is asked to log goes to stderr.
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            del os.environ["NCCL_DEBUG"]
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    n, d = wl["n"], wl["d"]
    ld = -(-d // 64) * 64
    sj = SelfJoin(local_rank)
    sj.set_stream(torch.cuda.current_stream().cuda_stream)
    if args.band_tiles:
        sj.set_option("band_tiles", args.band_tiles)
    if args.cta_pair >= 0:
        sj.set_option("cta_pair", args.cta_pair)
    for opt in args.option:
        k, v = opt.split("=", 1)
        sj.set_option(k, int(v))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def allmax(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    def allsum(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t)
        return float(t[0])

    # ---- dataset: generated on rank 0's GPU, replicated by the one broadcast --------------------
    # (rows padded to world equal bands so that the end-to-end leg can all-gather in place)
    dev_pts = torch.zeros((world * rows_per_band(n, world) if world > 1 else n, ld), dtype=torch.float16, device="cuda")
    if rank == 0:
        fill_device(sj, dev_pts, wl)
    if world > 1:
        dist.broadcast(dev_pts.view(torch.uint8), src=0)
    torch.cuda.synchronize()
    sj.set_points_device(dev_pts.data_ptr(), n, d, ld, keepalive=dev_pts)

    # ---- epsilon ------------------------------------------------------------------------------
    eps = wl["eps"]
    tuned_mean = None
    if eps is None:
        if rank == 0:
            eps, tuned_mean = sj.estimate_epsilon(wl["target"], 8192, 0.01)
        if world > 1:
            t = torch.tensor([eps if rank == 0 else 0.0], dtype=torch.float64, device="cuda")
            dist.broadcast(t, src=0)
            eps = float(t.item())
    per_point = int(wl.get("pairs_per_point", 256))

    # ---- the split over the GPUs --------------------------------------------------------------------
    # N > 1: the ranks take chunks of whole raster bands from one shared table, each whenever its join
    # stream has room (dealt_self_join): a GPU that runs faster under its own power cap takes more chunks,
    # so all ranks finish within one small chunk of each other.  --no-balance: one fixed, equal band per rank.
    dealt = world > 1 and not args.no_balance
    bounds = [band_bounds(n, world, r) for r in range(world)]
    cap_rows = int(max(b - a for a, b in bounds) * (1.3 if dealt else 1.0)) + 128
    capacity = max(1, cap_rows) * per_point
    table = SharedChunkTable.collective(n) if dealt else None

    def step_resident():
        if dealt:
            return dealt_self_join(sj, n, eps, table, None, capacity=capacity, flags=JOIN_NO_SORT)[2]
        a, b = bounds[rank]
        return sj.join(eps, q_begin=a, q_end=b, capacity=capacity, flags=JOIN_NO_SORT)

    for _ in range(args.warmup):
        step_resident()
    q_begin, q_end = bounds[rank]

    # ---- timed region 1: dataset resident, device-timed -----------------------------------------
    sampler = ClockSampler(local_rank)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    join_ms, norm_ms, found = [], [], 0
    cyc, tiles0 = [], 0
    barrier()
    sampler.start()
    ev0.record()
    for _ in range(args.steps):
        st = step_resident()
        join_ms.append(st.join_ms)
        norm_ms.append(st.norms_ms)
        found = int(st.pairs_found)
        cyc.append(int(st.cta0_cycles))
        tiles0 = int(st.cta0_tiles)
        setup_cyc, release_cyc = int(st.cta0_setup_cycles), int(st.cta0_release_cycles)
        feed_cyc, acc_cyc = int(st.cta0_feed_wait_cycles), int(st.cta0_acc_wait_cycles)
        last_rows = int(st.tiles_m) * 128
    ev1.record()
    barrier()
    clocks = sampler.stop()
    band_rows = min(last_rows, n) if dealt else q_end - q_begin  # query rows this rank joined in its last step
    rows_share = None
    if world > 1:
        t = torch.empty(world, dtype=torch.float64, device="cuda")
        dist.all_gather_into_tensor(t, torch.tensor([float(band_rows)], dtype=torch.float64, device="cuda"))
        rows_share = [int(x) for x in t.tolist()]
    total_ms = allmax(ev0.elapsed_time(ev1))
    found_total = int(allsum(float(found)))
    join_ms_max, norm_ms_max = allmax(float(np.mean(join_ms))), allmax(float(np.mean(norm_ms)))
    join_ms_min = -allmax(-float(np.mean(join_ms)))
    ms_per_step = total_ms / args.steps
    flop = 2.0 * n * n * d
    value = flop / (ms_per_step * 1e-3) / 1e12

    # ---- extra leg: symmetric schedule (each unordered pair computed once, both orientations
    # emitted; bit-identical output).  Reported beside the headline, never as the headline: the
    # metric still divides 2*N*N*D by the time although about half of those flops are executed.
    # At N > 1 rank r takes the raster bands r, 2G-1-r, 2G+r, ... of the triangle (balanced); the
    # all-to-all of pair records that follows it (fasted_b200/dist.py) is outside this interval, as
    # the sort is outside the headline interval.
    symmetric = None
    if not args.no_extras:
        sym_cap = max(capacity, n * per_point // world * 2)
        for _ in range(min(args.warmup, 1)):
            sj.join_symmetric_shard(eps, rank, world, capacity=sym_cap, flags=JOIN_NO_SORT)
        barrier()
        ev0.record()
        sym_found = 0
        for _ in range(args.steps):
            st = sj.join_symmetric_shard(eps, rank, world, capacity=sym_cap, flags=JOIN_NO_SORT)
            sym_found = int(st.pairs_found)
        ev1.record()
        barrier()
        sym_ms = allmax(ev0.elapsed_time(ev1)) / args.steps
        sym_found = int(allsum(float(sym_found)))
        symmetric = {"value": flop / (sym_ms * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": sym_ms,
                     "pairs_found": sym_found, "same_pair_count_as_full": sym_found == found_total,
                     "note": "2*N*N*D / time with the symmetric schedule; executed tensor flops are about half"}

    # ---- extra leg: accuracy against an FP64 brute-force join on a band of query rows ------------
    accuracy = None
    if rank == 0 and not args.no_extras:
        accuracy = accuracy_leg(sj, dev_pts, n, d, eps, per_point)

    # ---- timed region 2: end to end with host buffers -------------------------------------------
    e2e = None
    if not args.no_e2e:
        # Every step: the dataset comes from pinned HOST memory, the sorted pair list ends in HOST memory.
        # N = 1: fasted_set_points_host_f16, then fasted_join_stream, whose sort and device-to-host copy run
        # chunk by chunk behind the join, into one pinned buffer.  N > 1: every rank holds its own band of rows
        # on the host (the data-parallel loader: G host links in parallel), uploads it, ONE in-place NCCL
        # all-gather completes the matrix on every GPU; every rank joins its band (sort pipelined behind the
        # join), the per-rank counts are exchanged, and every rank's list lands in ONE shared, page-locked
        # host buffer at its exclusive-scan offset: the global row-major list, assembled without a copy.
        pad_begin = rank * rows_per_band(n, world) if world > 1 else 0
        pad_end = pad_begin + rows_per_band(n, world) if world > 1 else n
        host_pts = torch.empty((pad_end - pad_begin, ld), dtype=torch.float16).pin_memory()
        host_pts.copy_(dev_pts[pad_begin:pad_end])
        torch.cuda.synchronize()
        out_cap = int(min(n * per_point, max(1 << 20, int(1.05 * found_total) + 1024)))
        engine = GpuBandEngine(sj)
        engine.capacity_per_row = per_point
        engine.capacity_rows = cap_rows
        if world == 1:
            host_out = torch.empty((out_cap, 2), dtype=torch.int32).pin_memory()
            shared = None
        else:
            shared = SharedPairBuffer.collective(out_cap, register_cuda=True)

        def step_e2e():
            if world == 1:
                sj.set_points_ptr(host_pts.data_ptr(), n, d, ld)
                if args.e2e_mode == "serial":
                    st = sj.join(eps, capacity=capacity)
                    m = min(int(st.pairs_stored), out_cap)
                    sj.pairs_into(host_out.data_ptr(), m)
                    return st, m
                st = sj.join_stream(eps, capacity=capacity, pairs_host=host_out.data_ptr(), host_capacity=out_cap)
                return st, min(int(st.pairs_stored), out_cap)
            if dealt and args.join_behind_load:
                _, _, st = load_and_join(sj, dev_pts, host_pts, n, d, eps, table, shared, capacity=capacity,
                                         pieces=max(1, args.loader_pieces), lead_rows=args.lead_rows)
                return st, int(st.pairs_stored)
            if args.loader_pieces > 1:
                upload_and_allgather(dev_pts, host_pts, rank, world, pieces=args.loader_pieces)
            else:
                dev_pts[pad_begin:pad_end].copy_(host_pts, non_blocking=True)
                allgather_points(dev_pts, rank, world)
            sj.set_points_device(dev_pts.data_ptr(), n, d, ld, keepalive=dev_pts)
            if dealt:
                _, _, st = dealt_self_join(sj, n, eps, table, shared, capacity=capacity)
                return st, int(st.pairs_stored)
            _, _, stored = sharded_self_join(engine, n, eps, gather=False, bounds=bounds, shared=shared)
            return engine.last_stats, stored

        e2e_warm = min(args.warmup, 1)
        for _ in range(e2e_warm):
            step_e2e()
        barrier()
        t0 = time.perf_counter()
        ev0.record()
        copied = 0
        e2e_join_ms, e2e_tail_ms, e2e_chunks = [], [], 0
        for _ in range(args.steps):
            st, copied = step_e2e()
            e2e_join_ms.append(st.join_ms)
            e2e_tail_ms.append(st.tail_ms)
            e2e_chunks = int(st.chunks)
        ev1.record()
        barrier()
        wall_ms = (time.perf_counter() - t0) * 1e3
        e2e_ms = allmax(max(ev0.elapsed_time(ev1), wall_ms)) / args.steps
        d2h = int(allsum(float(copied * 8)))  # byte counts are whole-job totals, like the value
        e2e = {"value": flop / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": host_pts.numel() * 2 * world, "d2h_bytes_per_step": d2h,
               "join_kernel_ms": float(np.mean(e2e_join_ms)), "egress_tail_ms": float(np.mean(e2e_tail_ms)),
               "sort_ms": float(st.sort_ms), "mode": args.e2e_mode if world == 1 else "stream",
               "join_launches_per_step": e2e_chunks,
               "join_behind_load": bool(world > 1 and dealt and args.join_behind_load),
               "loader_pieces": args.loader_pieces if world > 1 else None,
               "api": "fasted_set_points_host_f16 + fasted_join_stream (pinned host buffers; sort and device-to-host "
                      "copy pipelined behind the join)"
               if world == 1 else ("per rank: pinned host band -> its GPU and NCCL all-gather piece by piece on side "
                                     "streams while fasted_join_stream_arriving already joins the first chunks of the "
                                     "rank's own band against the pieces that are there; then "
                                     if dealt and args.join_behind_load else
                                     "per rank: pinned host band -> its GPU, one NCCL all-gather, then ")
                                    + ("fasted_join_stream_shared: chunks taken from one shared table, every sorted chunk "
                                       "copied to its final place in one shared page-locked host buffer while the join runs"
                                       if dealt else "fasted_join_stream on the rank's band, count exchange, fasted_get_pairs "
                                       "into one shared page-locked host buffer at the exclusive-scan offset")
                                    + "; byte counts are sums over the ranks"}
        if shared is not None:
            # the single list on the host: strictly ascending keys == every band in place, nothing missing
            if rank == 0:
                k = shared.array[:min(found_total, out_cap)].astype(np.int64)
                keys = (k[:, 0] << 32) | k[:, 1]
                e2e["single_host_list_sorted"] = bool((np.diff(keys) > 0).all()) and len(keys) == found_total
                del k, keys
            barrier()
            shared.close()
        if world == 1:
            sj.set_points_device(dev_pts.data_ptr(), n, d, ld, keepalive=dev_pts)

    # ---- the reference's own kernels on the same GPU and buffer (N = 1 only, outside all timing) ------
    reference_gpu = None
    if rank == 0 and world == 1 and not args.no_refgpu:
        reference_gpu = reference_gpu_leg(SelfJoin, dev_pts, wl, eps, 100_000)

    # ---- CPU baseline on rank 0, N = 1 only ------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        import oracle
        q_rows, c_rows = size_cpu_sample(wl, budget_flop=1e12 * oracle.num_threads() / 16)
        sample = dev_pts[:c_rows, :d].contiguous().cpu().numpy().view(np.uint16)
        cpu = cpu_fp64_sample(sample, d, eps, q_rows)

    if rank == 0:
        peaks = _peaks()
        band_flop = 2.0 * band_rows * n * d  # rank 0's launch
        achieved = band_flop / (float(np.mean(join_ms)) * 1e-3) / 1e12
        peak = peaks["sustained"] if float(np.mean(join_ms)) > 500.0 else peaks["burst"]
        line = {
            "metric": "self_join_tflops", "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (value / PUBLISHED_A100_TFLOPS[name]) if name in PUBLISHED_A100_TFLOPS and not (args.points or args.dims) and world == 1 else None,
            "dtype": "f16xf16->f32", "data": "synthetic",
            "config": {
                "workload": f"{name}: self-join of {n} x {d} points, {wl['dist']} (seed {SEED}), FP16, "
                            f"eps for ~{wl['target']} neighbours per point",
                "n": n, "d": d, "epsilon": eps, "mean_neighbours": (found_total - n) / n,
                "parallelism": (f"query rows over {world} GPUs: " + ("chunks of raster bands taken on demand from a shared "
                                "table" if dealt else "one fixed equal band per rank")) if world > 1 else "single GPU",
                "rows_per_rank_last_step": rows_share,
                "rank0_cpu_cores": (f"{len(numa_cores)} cores next to its GPU" if numa_cores else None),
                "l2": "inputs larger than L2 (no flush needed)" if n * ld * 2 > 2 * 126e6 else "inputs fit L2",
                "baseline_note": "vs_baseline divides by the reference's published A100-PCIe figure for this shape "
                                 "(153.64 TFLOPS at eps=0.001)" if name in PUBLISHED_A100_TFLOPS else None,
            },
            "pairs_found": found_total, "pairs_per_s": found_total / (ms_per_step * 1e-3),
            "frac_of_nominal_fp16_peak": value / (NOMINAL_FP16_TFLOPS * world),
            "kernel_ms": {"join": join_ms_max, "join_fastest_rank": join_ms_min, "norms": norm_ms_max},
            "clocks": clocks,
            # from the kernel's own cycle counter (CTA 0): mean SM clock of the join launches and the share of
            # CTA 0's cycles that its tiles' tensor work needs at full rate (k_steps x 4 MMAs x 128 clocks a tile)
            "sm_clock_in_kernel_mhz": float(np.mean(cyc)) / (float(np.mean(join_ms)) * 1e3) if cyc and cyc[0] else None,
            "tensor_busy_share_cta0": (tiles0 * (-(-d // 64)) * 512.0) / float(np.mean(cyc)) if cyc and cyc[0] else None,
            "cta0_cycles": {"tiles": float(np.mean(cyc)) if cyc else None, "setup": setup_cyc, "tmem_release": release_cyc,
                            "mma_thread_waited_for_operands": feed_cyc, "mma_thread_waited_for_accumulator": acc_cyc},
            "e2e": e2e,
            "gpu_launches": 2 * args.steps,  # per step: row_norms_kernel, join_kernel (records stay packed until asked for)
            "roofline": {"bound": "tensor", "kernel": "join_kernel", "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s", "frac": achieved / peak if peak else None,
                         # DRAM bytes per launch: ncu measured one pass over the candidates per raster band
                         # (17.09 GB at 16 tile rows per band, 8.55 GB at 32, on 65,536 x 4096); scaled by that
                         # rule to this launch (bands of 16 tile rows).
                         "traffic": float(-(-(-(-band_rows // 128)) // (args.band_tiles or 16)) * n * ld * 2 + band_rows * ld * 2),
                         "traffic_source": "ncu dram__bytes_read.sum of a 65536 x 4096 launch, scaled by bands x N*D*2",
                         "peak_source": f"{peaks['source']} cuBLAS bf16 "
                                        f"({'sustained' if float(np.mean(join_ms)) > 500.0 else 'burst'})",
                         "norms_kernel": {"bound": "hbm", "achieved": (n * ld * 2 + n * 4) / (float(np.mean(norm_ms)) * 1e-3) / 1e9,
                                          "peak": peaks["hbm"], "unit": "GB/s"}},
            "cpu_baseline": cpu,
            "reference_gpu": reference_gpu,
            "symmetric": symmetric,
            "accuracy_vs_fp64": accuracy,
        }
        if tuned_mean is not None:
            line["config"]["epsilon_tuned"] = True
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    sj.close()


def accuracy_leg(sj, dev_pts, n: int, d: int, eps: float, per_point: int) -> dict:
    """Pair set and distances of a band of query rows against an FP64 brute-force join on the device (the
    reference's accuracy tables report the same two figures: per-point IoU and signed distance error)."""
    import torch
    from fasted_b200 import JOIN_DIST2
    a_rows = min(256, n)
    q0 = max(0, (n // 2) // 128 * 128)
    q0 = min(q0, n - a_rows)
    cap = a_rows * max(8192, 4 * per_point)
    sj.join(eps, q_begin=q0, q_end=q0 + a_rows, capacity=cap, flags=JOIN_DIST2)
    got, got_d2 = sj.pairs(with_dist2=True)
    rows = np.arange(q0, q0 + a_rows, dtype=np.int32)
    _, truth = sj.brute_force_pairs(rows, eps, capacity=cap)
    kg = (got[:, 0].astype(np.int64) << 32) | got[:, 1].astype(np.int64)
    kt = (truth[:, 0].astype(np.int64) << 32) | truth[:, 1].astype(np.int64)
    inter = np.intersect1d(kg, kt, assume_unique=True)
    cg = np.bincount(got[:, 0] - q0, minlength=a_rows)
    ct = np.bincount(truth[:, 0] - q0, minlength=a_rows)
    ci = np.bincount((inter >> 32) - q0, minlength=a_rows)
    union = cg + ct - ci
    iou = np.where(union > 0, ci / np.maximum(union, 1), 1.0)
    off = got[:, 0] != got[:, 1]
    gi = torch.from_numpy(got[off].astype(np.int64)).cuda()
    d64 = torch.empty(gi.shape[0], dtype=torch.float64, device="cuda")
    for a in range(0, gi.shape[0], 4096):
        xa = dev_pts[gi[a:a + 4096, 0], :d].double()
        xb = dev_pts[gi[a:a + 4096, 1], :d].double()
        d64[a:a + 4096] = ((xa - xb) ** 2).sum(dim=1).sqrt()
    d32 = np.sqrt(np.maximum(got_d2[off].astype(np.float64), 0.0))
    err = d32 - d64.cpu().numpy()
    # the same band with correctly rounded norms (option exact_norms; not the reference's numerics)
    sj.set_option("exact_norms", 1)
    sj.join(eps, q_begin=q0, q_end=q0 + a_rows, capacity=cap)
    got2 = sj.pairs()
    sj.set_option("exact_norms", 0)
    sj.row_norms_timed()
    k2 = (got2[:, 0].astype(np.int64) << 32) | got2[:, 1].astype(np.int64)
    inter2 = np.intersect1d(k2, kt, assume_unique=True)
    c2 = np.bincount(got2[:, 0] - q0, minlength=a_rows)
    ci2 = np.bincount((inter2 >> 32) - q0, minlength=a_rows)
    un2 = c2 + ct - ci2
    iou2 = np.where(un2 > 0, ci2 / np.maximum(un2, 1), 1.0)
    return {"query_rows": [int(q0), int(q0 + a_rows)], "pairs_ours": int(len(kg)), "pairs_fp64": int(len(kt)),
            "with_exact_norms_option": {"pairs": int(len(k2)), "mean_per_point_iou": float(iou2.mean())},
            "mean_per_point_iou": float(iou.mean()), "min_per_point_iou": float(iou.min()),
            "distance_error_mean": float(err.mean()) if len(err) else 0.0,
            "distance_error_std": float(err.std()) if len(err) else 0.0,
            "truth": "FP64 direct-form brute force on the GPU (plain CUDA cores) over the same FP16 inputs"}


if __name__ == "__main__":
    main()
