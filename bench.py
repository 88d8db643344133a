"""Benchmark of the fused FP8 paged EXTEND/prefill attention path.

    python bench.py --gpus N --steps K --warmup W            # this library, on N B200s
    python bench.py --impl reference --steps K --warmup W    # the reference's own CPU oracle on host cores

Workload (`config.workload` = "c2_main_24x4"): the main D256 GQA 24:4 profile -- per GPU 8
requests, prefix ~ U{1024..8192}, 2048 extend tokens each, BF16 K/V pools of 446 464 slots
addressed through one shuffled page table, 16 layers = 16 distinct pool pairs resident in HBM
(29.3 GB), replayed back to back.  One STEP = all 8 requests through all 16 layers: 16 calls of the
batched entry `akl_prefill_extend_batch` (four launches each).  Values ~ N(0,1) with 2 % of
channels x16 (seeded, synthetic).

metric   inclusive TF/s: attention FLOPs 4*Hq*D*T*(prefix + (T+1)/2) per request-layer
         (reference bench/candidate_bench.py:210-212) over ONE span holding everything the
         operator does from BF16 inputs to BF16 output (gather, statistics, transform,
         attention, output write; reference bench/candidate_bench.py:876-898).
value    inputs already resident in HBM, timed with CUDA events on the launch stream,
         max over ranks.
e2e      the same metric through `prefill_extend_batch` with HOST buffers: per layer one pinned
         staging buffer (the 8 query chunks and their new K/V rows) goes to the device in one copy,
         the K/V rows enter the paged pool as in a serving engine, the batch runs, and the BF16
         outputs go back to pinned host memory in one copy; copies overlap compute on their own
         streams over three slots.
roofline the attention launch alone against the dense-FP8 tensor peak (measured in this run with a
         library FP8 GEMM; 2x the measured BF16 peak of MEASURED_PEAKS.json and the vendor nominal
         are reported beside it), and the preprocessing launches against the measured HBM copy
         bandwidth.
c5_serving   the 256-request serving-shaped batch (extend ~ geometric mean 128 capped at 512, prefix ~
         U{0..32768}) as one CUDA graph of one batched call, replayed; with N GPUs the requests are
         dealt to the ranks by attended pairs.
cpu_baseline / --impl reference   the UNMODIFIED reference's CPU oracle (`oracle_a.reference`, and the
         FP8-QK composition of its `quant` + `oracle_a.attention`) from oracle/_ref on configuration 1
         (256 cached + 64 new tokens, 24:4, 4096-slot pool), all host threads; where oracle/_ref is
         missing, the oracle port (oracle/akl_oracle.py) on the same configuration.
gpu_reference    the reference's own operator (its mma.sync kernel built for sm_100a) on one request
         of the workload, same box, when its prebuilt extension is present in oracle/_ref.
With N > 1 each rank runs its own 8-request workload (requests are independent units; no
data-path collective): weak scaling, value = all ranks' FLOPs / slowest rank's time.  The line
then also carries `strong_c2` (the 8 requests dealt 8/N per rank) and `kv_split` (the long single
request cut along the KV axis over the N ranks: parity against the split-composed oracle on a small
case, then the 131 072 + 8 192 configuration timed phase by phase).
"""
from __future__ import annotations

import argparse
import datetime
import ctypes
import json
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

HQ, HKV, D = 24, 4, 256
POOL_ROWS = 446_464
LAYERS = 16
REQUESTS = 8
QK_I8 = False          # --qk int8 runs the reference's default INT8-QK mode instead of FP8-QK
T_EXT = 2048
SM_SCALE = 1.0 / 16.0
NOMINAL_FP8_TFLOPS = 4500.0
KERNELS_PER_BATCH = 4         # tile statistics + Q quantise, means + scales, K/V transform, attention
REF_DIR = ROOT / "oracle" / "_ref"


def flops(prefix: int, t: int, hq: int = HQ) -> float:
    return 4.0 * hq * D * t * (prefix + (t + 1) / 2.0)


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text())
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "fallback": True}


# --------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while a region runs
    (one long-lived `nvidia-smi -lms 50` child, stopped when the region ends)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self._proc = None
        self._thread = None

    def _drain(self):
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.strip().split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def __enter__(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._thread = threading.Thread(target=self._drain, daemon=True)
            self._thread.start()
            time.sleep(0.3)                      # first samples land before the region starts
            self.samples.clear()
        except OSError:
            self._proc = None
        return self

    def __exit__(self, *exc):
        if self._proc is not None:
            self._proc.terminate()               # the exact child started above
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
            self._thread.join(timeout=5)

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, flag in zip(names, s[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def device_time(torch, fn, reps: int, warm: int = 2) -> float:
    """Mean milliseconds per call of `fn` (CUDA events on the current stream, after warm-up)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def capture(torch, fn):
    """`fn` captured once into a CUDA graph; returns the replay callable."""
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    return graph.replay


# --------------------------------------------------------------------------------------
# main workload
# --------------------------------------------------------------------------------------
def outlier_device(torch, g, dev, shape, seed, dtype=None):
    g.manual_seed(seed)
    x = torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
    mask = torch.rand(D, generator=g, device=dev) < 0.02
    mask[seed % D] = True
    x[..., mask] *= 16.0
    return x.to(dtype or torch.bfloat16)


def build_workload(torch, syn, dev, rank: int, lens=None, layers=None):
    """Device-resident pools, page tables and queries of one rank (seeded per object)."""
    g = torch.Generator(device=dev)
    layers = LAYERS if layers is None else layers
    cfg = 2 + 100 * rank                                   # distinct values and page tables per rank
    # the request lengths are those of rank 0 on every rank: weak scaling means the same work per GPU
    lens = syn.c2_lengths(REQUESTS, seed=syn.object_seed(2, 0, 4)) if lens is None else lens
    gcpu = torch.Generator().manual_seed(syn.object_seed(cfg, 0, 3))
    table = torch.randperm(POOL_ROWS, generator=gcpu).to(dev)
    k_pools, v_pools = [], []
    for layer in range(layers):                            # chunked fill keeps the fp32 temporary small
        kp = torch.empty((POOL_ROWS, HKV, D), dtype=torch.bfloat16, device=dev)
        vp = torch.empty((POOL_ROWS, HKV, D), dtype=torch.bfloat16, device=dev)
        step = POOL_ROWS // 8
        for c in range(8):
            kp[c * step:(c + 1) * step] = outlier_device(torch, g, dev, (step, HKV, D), syn.object_seed(cfg, c, 1, layer))
            vp[c * step:(c + 1) * step] = outlier_device(torch, g, dev, (step, HKV, D), syn.object_seed(cfg, c, 2, layer))
        k_pools.append(kp)
        v_pools.append(vp)
    reqs, off = [], 0
    total_t = sum(t for _, t in lens)
    q_all = [torch.empty((total_t, HQ, D), dtype=torch.bfloat16, device=dev) for _ in range(layers)]
    out_all = [torch.empty((total_t, HQ, D), dtype=torch.bfloat16, device=dev) for _ in range(layers)]
    row = 0
    for i, (prefix, t) in enumerate(lens):
        n = prefix + t
        for layer in range(layers):
            q_all[layer][row:row + t] = outlier_device(torch, g, dev, (t, HQ, D), syn.object_seed(cfg, i, 0, layer))
        reqs.append({"prefix": prefix, "T": t, "N": n, "row0": row, "idx": table[off:off + n].contiguous()})
        off += n
        row += t
    return {"k_pools": k_pools, "v_pools": v_pools, "reqs": reqs, "q_all": q_all, "out_all": out_all,
            "layers": layers, "flops_per_step": sum(flops(r["prefix"], r["T"]) for r in reqs) * layers,
            "tokens_per_step": sum(r["T"] for r in reqs)}


def layer_requests(wl, layer, q=None, out=None):
    q = wl["q_all"][layer] if q is None else q
    out = wl["out_all"][layer] if out is None else out
    kp, vp = wl["k_pools"][layer], wl["v_pools"][layer]
    return [{"q": q[r["row0"]:r["row0"] + r["T"]], "k_pool": kp, "v_pool": vp, "idx": r["idx"],
             "prefix": r["prefix"], "out": out[r["row0"]:r["row0"] + r["T"]]} for r in wl["reqs"]]


class Stepper:
    """One pass of the workload: layer l goes through batch workspace l % lanes on side stream
    l % lanes (event fork/join), so the gather/quantise launches of one layer fill the SMs that
    the attention launch of the previous layer leaves as its work list drains."""

    def __init__(self, torch, pkg, wl, dev, lanes: int):
        self.torch, self.wl = torch, wl
        total_n = sum(r["N"] for r in wl["reqs"])
        total_t = sum(r["T"] for r in wl["reqs"])
        self.lanes = max(1, lanes)
        self.ws = [pkg.plan_batch_workspace(dev, max_requests=len(wl["reqs"]), max_total_kv_len=total_n,
                                            max_total_q_len=total_t, q_heads=HQ, kv_heads=HKV)
                   for _ in range(self.lanes)]
        self.plans = [self.ws[l % self.lanes].plan(layer_requests(wl, l), sm_scale=SM_SCALE, qk_i8=QK_I8)
                      for l in range(wl["layers"])]
        self.streams = [torch.cuda.Stream(device=dev) for _ in range(self.lanes)]

    def __call__(self):
        torch = self.torch
        if self.lanes == 1:
            for l, plan in enumerate(self.plans):
                self.ws[0].launch(plan)
            return
        main = torch.cuda.current_stream()
        fork = torch.cuda.Event()
        fork.record(main)
        for s in self.streams:
            s.wait_event(fork)
        for l, plan in enumerate(self.plans):
            with torch.cuda.stream(self.streams[l % self.lanes]):
                self.ws[l % self.lanes].launch(plan)
        for s in self.streams:
            join = torch.cuda.Event()
            join.record(s)
            main.wait_event(join)

    def status(self):
        return [w.status() for w in self.ws]


def phase_rooflines(torch, K, stepper, wl, peaks, fp8_peak):
    """Device time of each launch of layer 0's batch, alone on the GPU, against its roofline."""
    ws, plan = stepper.ws[0], stepper.plans[0]
    ws.launch(plan)
    torch.cuda.synchronize()
    ms = {}
    for name, mask in (("stats", K.AKL_BATCH_STATS), ("means", K.AKL_BATCH_MEANS),
                       ("transform", K.AKL_BATCH_TRANSFORM), ("attention", K.AKL_BATCH_ATTENTION)):
        ms[name] = device_time(torch, lambda: ws.launch(plan, phases=mask, upload=False), reps=10)
    reqs = wl["reqs"]
    sum_n, sum_t = sum(r["N"] for r in reqs), sum(r["T"] for r in reqs)
    kv_rows = 2 * sum_n * HKV * D * 2                      # one read of the request's K and V rows
    bytes_ = {"stats": kv_rows + sum_n * 8,                                           # K and V rows once + page table
              # the rows again, K8 + V8 write, page table; Q read and Q8 write (the Q quantisation runs in this launch)
              "transform": kv_rows + 2 * sum_n * HKV * D + sum_n * 8 + sum_t * HQ * D * 3}
    attn_flops = sum(flops(r["prefix"], r["T"]) for r in reqs)
    achieved = attn_flops / ms["attention"] / 1e9
    peak = fp8_peak if fp8_peak else 2.0 * peaks["bf16_tflops"]
    traffic = traffic_note = None
    tpath = ROOT / "profiles" / "attn_sm100_traffic.json"
    if tpath.exists():
        cap = json.loads(tpath.read_text())
        # the capture covers two requests (a full-size launch is too large to profile); DRAM traffic
        # follows the units processed (Q8 + K8 + V8 + output bytes), so scale it to this launch
        units = sum(r["T"] * HQ * D + 2 * r["N"] * HKV * D + r["T"] * HQ * D * 2 for r in reqs)
        traffic = cap["dram_bytes_per_launch"] * units / cap["captured_units_bytes"]
        traffic_note = (f"ncu capture of a 2-request launch ({cap['dram_bytes_per_launch']} B) scaled by the "
                        f"units processed ({units} / {cap['captured_units_bytes']} B)")
    roof = {"bound": "tensor", "kernel": "attn_sm100_kernel (persistent, one launch per 8-request layer)",
            "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_note,
            "peak_source": ("measured FP8 E4M3 GEMM 8192^3 in this run (tensor library, burst)" if fp8_peak
                            else "2 x measured BF16 burst peak (MEASURED_PEAKS.json)"),
            "frac_of_2x_measured_bf16_burst": achieved / (2.0 * peaks["bf16_tflops"]),
            "frac_of_2x_measured_bf16_sustained": achieved / (2.0 * peaks["bf16_tflops_sustained"]),
            "frac_of_nominal_dense_fp8": achieved / NOMINAL_FP8_TFLOPS,
            "attention_ms_per_launch": ms["attention"], "flops_per_launch": attn_flops,
            "prep": {name: {"ms_per_launch": ms[name], "algorithmic_bytes": bytes_[name],
                            "achieved": bytes_[name] / ms[name] / 1e6, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": bytes_[name] / ms[name] / 1e6 / peaks["hbm_gbs"]}
                     for name in ("stats", "transform")},
            "means_ms_per_launch": ms["means"]}
    return roof


def measure_fp8_gemm_peak(torch, dev):
    """Dense FP8 (E4M3) GEMM 8192^3 through the tensor library: the roofline denominator only."""
    try:
        n = 8192
        a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()
        one = torch.tensor(1.0, device=dev)
        for _ in range(3):
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        best = 1e9
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(10):
            e0.record()
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2.0 * n ** 3 / best / 1e9
    except Exception:  # noqa: BLE001 - the denominator falls back to 2x measured BF16
        return None


def measure_pinned_copy(torch, dev, nbytes: int = 256 << 20):
    """Achievable pinned-host copy bandwidth (GB/s) in each direction, alone."""
    host = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    devb = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    h2d = device_time(torch, lambda: devb.copy_(host, non_blocking=True), reps=4)
    d2h = device_time(torch, lambda: host.copy_(devb, non_blocking=True), reps=4)
    return nbytes / h2d / 1e6, nbytes / d2h / 1e6


def time_e2e(torch, pkg, wl, dev, steps: int, warmup: int, slots_n: int = 3):
    """Host buffers in, host buffers out, through the public batched entry point."""
    reqs = wl["reqs"]
    total_t = sum(r["T"] for r in reqs)
    total_n = sum(r["N"] for r in reqs)
    q_bytes, kv_bytes = total_t * HQ * D * 2, total_t * HKV * D * 2
    in_bytes = q_bytes + 2 * kv_bytes
    new_rows = torch.cat([r["idx"][r["prefix"]:] for r in reqs])      # pool rows the chunk's K/V go to
    host_in = torch.randn(in_bytes // 2).to(torch.bfloat16).pin_memory()   # q | k | v of one layer, contiguous
    host_out = [torch.empty((total_t, HQ, D), dtype=torch.bfloat16).pin_memory() for _ in range(slots_n)]
    slots = []
    for _ in range(slots_n):
        stage = torch.empty(in_bytes // 2, dtype=torch.bfloat16, device=dev)
        slots.append({
            "stage": stage, "q": stage[:q_bytes // 2].view(total_t, HQ, D),
            "k": stage[q_bytes // 2:(q_bytes + kv_bytes) // 2].view(total_t, HKV, D),
            "v": stage[(q_bytes + kv_bytes) // 2:].view(total_t, HKV, D),
            "out": torch.empty((total_t, HQ, D), dtype=torch.bfloat16, device=dev),
            "ws": pkg.plan_batch_workspace(dev, max_requests=len(reqs), max_total_kv_len=total_n,
                                           max_total_q_len=total_t, q_heads=HQ, kv_heads=HKV),
            "loaded": torch.cuda.Event(), "computed": torch.cuda.Event(), "drained": torch.cuda.Event()})
    h2d, d2h, compute = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
    h2d_bytes = in_bytes * wl["layers"]
    d2h_bytes = total_t * HQ * D * 2 * wl["layers"]

    def one_step():
        for layer in range(wl["layers"]):
            s = slots[layer % slots_n]
            kp, vp = wl["k_pools"][layer], wl["v_pools"][layer]
            with torch.cuda.stream(h2d):
                h2d.wait_event(s["computed"])                     # slot inputs free again
                s["stage"].copy_(host_in, non_blocking=True)      # ONE copy per layer
                s["loaded"].record(h2d)
            compute.wait_event(s["loaded"])
            compute.wait_event(s["drained"])                      # slot output copied out
            kp.index_copy_(0, new_rows, s["k"])                   # the chunk's K/V enter the paged pool
            vp.index_copy_(0, new_rows, s["v"])
            pkg.prefill_extend_batch(layer_requests(wl, layer, q=s["q"], out=s["out"]), workspace=s["ws"],
                                     sm_scale=SM_SCALE, qk_i8=QK_I8)
            s["computed"].record(compute)
            with torch.cuda.stream(d2h):
                d2h.wait_event(s["computed"])
                host_out[layer % slots_n].copy_(s["out"], non_blocking=True)   # ONE copy per layer
                s["drained"].record(d2h)
        compute.wait_stream(d2h)

    for _ in range(max(1, min(warmup, 2))):
        one_step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one_step()
    e1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    return max(e0.elapsed_time(e1) / 1e3, wall) / steps, h2d_bytes, d2h_bytes


# --------------------------------------------------------------------------------------
# the 256-request serving-shaped batch
# --------------------------------------------------------------------------------------
def c5_serving(torch, dist, pkg, K, syn, dev, rank: int, world: int, peaks, reps: int = 5):
    from attn_kernel_lab_b200 import dist as D_

    lens_all = syn.c5_lengths(256)
    costs = [flops(p, t) for p, t in lens_all]
    mine = D_.partition_requests(costs, world)[rank]
    lens = [lens_all[i] for i in mine]
    total = sum(p + t for p, t in lens)
    slots = (int(total * 1.1) + 63) // 64 * 64
    g = torch.Generator(device=dev)
    kp = torch.empty((slots, HKV, D), dtype=torch.bfloat16, device=dev)
    vp = torch.empty((slots, HKV, D), dtype=torch.bfloat16, device=dev)
    step = (slots + 15) // 16
    for c in range(16):
        lo, hi = c * step, min(slots, (c + 1) * step)
        if lo < hi:
            kp[lo:hi] = outlier_device(torch, g, dev, (hi - lo, HKV, D), syn.object_seed(5, c, 1))
            vp[lo:hi] = outlier_device(torch, g, dev, (hi - lo, HKV, D), syn.object_seed(5, c, 2))
    g.manual_seed(syn.object_seed(5, 0, 3))
    perm = torch.randperm(slots, device=dev, generator=g)
    total_t = sum(t for _, t in lens)
    q_all = outlier_device(torch, g, dev, (total_t, HQ, D), syn.object_seed(5, 0, 0))
    out_all = torch.empty_like(q_all)
    reqs, at, row = [], 0, 0
    for p, t in lens:
        reqs.append({"q": q_all[row:row + t], "k_pool": kp, "v_pool": vp, "idx": perm[at:at + p + t].contiguous(),
                     "prefix": p, "out": out_all[row:row + t]})
        at += p + t
        row += t
    ws = pkg.plan_batch_workspace(dev, max_requests=len(reqs), max_total_kv_len=total, max_total_q_len=total_t,
                                  q_heads=HQ, kv_heads=HKV)
    plan = ws.plan(reqs, sm_scale=SM_SCALE, qk_i8=QK_I8)
    ws.launch(plan)
    torch.cuda.synchronize()
    replay = capture(torch, lambda: ws.launch(plan))
    ms_batch = device_time(torch, replay, reps=reps)
    phases = {}
    for name, mask in (("stats", K.AKL_BATCH_STATS), ("means", K.AKL_BATCH_MEANS),
                       ("transform", K.AKL_BATCH_TRANSFORM), ("attention", K.AKL_BATCH_ATTENTION)):
        phases[name] = device_time(torch, lambda: ws.launch(plan, phases=mask, upload=False), reps=3, warm=1)
    if ws.status() != 0:
        raise SystemExit("device status word set in the serving batch: no number reported")
    t = torch.tensor([ms_batch], device=dev, dtype=torch.float64)
    fl = torch.tensor([sum(flops(p, t_) for p, t_ in lens)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(fl, op=dist.ReduceOp.SUM)
    ms_max, fl_all = float(t.item()), float(fl.item())
    sum_n = sum(p + t_ for p, t_ in lens)
    kv_rows = 2 * sum_n * HKV * D * 2
    step_bytes = kv_rows + 2 * total_t * HQ * D * 2 + sum_n * 8
    prep_bytes = {"stats": kv_rows + sum_n * 8, "transform": kv_rows + 2 * sum_n * HKV * D + sum_n * 8 + total_t * HQ * D * 3}
    del kp, vp
    return {"requests": 256, "requests_this_rank": len(reqs), "partition": f"by request, attended pairs, x{world}",
            "launch": "one CUDA graph of one batched call (table copy + 4 launches), replayed",
            "ms_per_batch": ms_max, "tflops": fl_all / ms_max / 1e9,
            "tokens_per_s": sum(t_ for _, t_ in lens_all) / ms_max * 1e3,
            "launches_per_batch": KERNELS_PER_BATCH,
            "rank0": {"kv_tokens": sum_n, "extend_tokens": total_t, "phase_ms": phases,
                      "attention_tflops": sum(flops(p, t_) for p, t_ in lens) / phases["attention"] / 1e9,
                      "hbm_frac_of_prep": {name: prep_bytes[name] / phases[name] / 1e6 / peaks["hbm_gbs"]
                                           for name in ("stats", "transform")},
                      "hbm_frac_whole_batch": step_bytes / ms_batch / 1e6 / peaks["hbm_gbs"]}}


# --------------------------------------------------------------------------------------
# multi-GPU legs
# --------------------------------------------------------------------------------------
def strong_c2(torch, dist, pkg, syn, dev, rank: int, world: int, wl):
    """The 8 requests of ONE workload dealt over the ranks (layer 0's pools of this rank stand in)."""
    from attn_kernel_lab_b200 import dist as D_

    lens = syn.c2_lengths(REQUESTS, seed=syn.object_seed(2, 0, 4))
    parts = D_.partition_requests([flops(p, t) for p, t in lens], world)
    mine = [wl["reqs"][i] for i in parts[rank]]
    ms = 0.0
    if mine:
        ws = pkg.plan_batch_workspace(dev, max_requests=len(mine), max_total_kv_len=sum(r["N"] for r in mine),
                                      max_total_q_len=sum(r["T"] for r in mine), q_heads=HQ, kv_heads=HKV)
        all_reqs = layer_requests(wl, 0)
        plan = ws.plan([all_reqs[i] for i in parts[rank]], sm_scale=SM_SCALE, qk_i8=QK_I8)
        replay = capture(torch, lambda: ws.launch(plan))
        ms = device_time(torch, replay, reps=10)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total = sum(flops(p, t_) for p, t_ in lens)
    return {"scaling": "strong", "requests": REQUESTS, "layers": 1, "partition": [len(p) for p in parts],
            "ms_per_layer": float(t.item()), "tflops": total / float(t.item()) / 1e9}


def kv_split_leg(torch, dist, pkg, syn, dev, rank: int, world: int):
    """KV-axis split of one long request over the ranks: parity on a small case against the
    split-composed oracle (the checker, on rank 0), then the long-context configuration
    (32:4 heads, 131 072 cached + 8 192 new tokens) timed phase by phase with CUDA events."""
    import numpy as np

    from attn_kernel_lab_b200 import dist as D_

    result = {"world": world}
    # ---- parity: 24:4, 300 extend rows; every rank owns keys (one split granule each and a
    # ragged rest), so the case grows with the world size ---------------------------------
    T = 300
    N = D_.SPLIT_GRANULE * world + 476
    prefix = N - T
    q = syn.outlier_normal((T, HQ, D), 4411).to(torch.bfloat16)
    k = syn.outlier_normal((N, HKV, D), 4412).to(torch.bfloat16)
    v = syn.outlier_normal((N, HKV, D), 4413).to(torch.bfloat16)
    ranges = D_.kv_split_ranges(N, world)
    lo, hi = ranges[rank]
    ws = pkg.FP8PrefillWorkspace(dev)
    out, lse, (rlo, rhi) = D_.prefill_extend_kv_split(
        ws, q.to(dev), k.to(dev), v.to(dev), torch.arange(lo, hi, device=dev), prefix, n_total=N, kv_lo=lo,
        sm_scale=SM_SCALE, qk_i8=QK_I8)
    torch.cuda.synchronize()
    status = ws.status()
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rows": (rlo, rhi), "out": out.float().cpu().numpy(), "lse": lse.cpu().numpy(),
                                      "status": status})
    # rank 0 checks; whatever happens there, it goes on to the collectives below with the others
    if rank == 0:
      try:
        sys.path.insert(0, str(ROOT / "oracle"))
        import akl_oracle as O                      # the checker

        qf, kf, vf = q.float().numpy(), k.float().numpy(), v.float().numpy()
        qp = O.preprocess_q(qf, SM_SCALE, qk_i8=QK_I8)
        kvp = O.preprocess_kv(kf, vf, qk_i8=QK_I8)
        refs = [O.attention(qp, kvp, prefix, T, HQ // HKV, return_lse=True, kv_lo=a, kv_hi=b) for a, b in ranges]
        want_o, want_l = O.merge_splits([O.round_to_bf16(r[0]) for r in refs], [r[1] for r in refs])
        got_o, got_l = np.zeros_like(want_o), np.zeros_like(want_l)
        for part in gathered:
            a, b = part["rows"]
            got_o[a:b], got_l[a:b] = part["out"], part["lse"]
        d = (got_o.astype(np.float64) - want_o).reshape(-1, D)
        rel = np.linalg.norm(d, axis=1) / np.maximum(np.linalg.norm(want_o.reshape(-1, D).astype(np.float64), axis=1), 1e-30)
        result["parity"] = {"case": f"T={T} N={N} prefix={prefix} 24:4 over {world} KV parts, against the split-composed oracle",
                            "lse_max": float(np.abs(got_l - want_l).max()), "rowrel_median": float(np.median(rel)),
                            "rows_over_9e-3": int((rel > 9e-3).sum()), "rows": int(rel.size),
                            "status_words": [part["status"] for part in gathered]}
      except Exception as exc:                       # noqa: BLE001 - reported, not raised
        result["parity"] = {"error": f"{type(exc).__name__}: {exc}"}

    # ---- the long-context configuration, timed -------------------------------------------
    Hq4, T4, P4 = 32, 8192, 131072
    N4 = T4 + P4
    lo, hi = D_.kv_split_ranges(N4, world)[rank]
    n_local = hi - lo
    g = torch.Generator(device=dev)
    g.manual_seed(syn.object_seed(4, 0, 0))                  # the same queries and sink basis on every rank
    q4 = torch.randn((T4, Hq4, D), generator=g, device=dev)
    basis, _ = torch.linalg.qr(torch.randn((D, 8), generator=g, device=dev))
    w = torch.randn((4, 8), generator=g, device=dev)
    wbar = w.mean(dim=0)
    q4 = (q4 + 2.0 * (basis @ (wbar / wbar.norm()))[None, None, :]).to(torch.bfloat16)
    g.manual_seed(syn.object_seed(4, rank, 1))
    k4 = torch.randn((n_local, HKV, D), generator=g, device=dev)
    if lo == 0:
        k4[:4] += 4.0 * (w @ basis.T)[:, None, :]
    k4 = k4.to(torch.bfloat16)
    v4 = torch.randn((n_local, HKV, D), generator=g, device=dev).to(torch.bfloat16)
    # 64-slot runs of the local pool, runs permuted
    runs = (n_local + 63) // 64
    order = torch.randperm(runs, generator=torch.Generator().manual_seed(syn.object_seed(4, rank, 3)))
    idx_local = (order[:, None] * 64 + torch.arange(64)[None, :]).reshape(-1)[:n_local].to(dev)
    kp = torch.zeros((runs * 64, HKV, D), dtype=torch.bfloat16, device=dev)
    vp = torch.zeros_like(kp)
    kp[idx_local] = k4
    vp[idx_local] = v4
    del k4, v4
    ws4 = pkg.FP8PrefillWorkspace(dev)
    lib = K_load()
    marks = {}

    def span(name, fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        marks.setdefault(name, []).append((e0, e1))

    st = lambda: torch.cuda.current_stream(dev).cuda_stream   # noqa: E731

    def phases(name, call):
        from attn_kernel_lab_b200 import kernel as K_

        span(name, lambda: K_.check(getattr(lib, name)(ctypes.byref(call), st()), name))

    def ar_sum(t):
        span("stats_allreduce", lambda: dist.all_reduce(t, op=dist.ReduceOp.SUM))

    def ar_max(t):
        span("stats_allreduce", lambda: dist.all_reduce(t, op=dist.ReduceOp.MAX))

    def merge(parts_o, parts_l):
        res = []
        span("merge", lambda: res.append(D_.merge_states(parts_o, parts_l)))
        return res[0]

    def one_pass():
        marks.clear()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        o_i, l_i = D_.kv_split_local(ws4, q4, kp, vp, idx_local, P4, n_total=N4, kv_lo=lo, sm_scale=SM_SCALE,
                                     qk_i8=QK_I8, all_reduce_sum=ar_sum, all_reduce_max=ar_max, phases=phases)
        x0 = torch.cuda.Event(enable_timing=True)
        x0.record()
        out_r, lse_r, rows = D_.exchange_and_merge(o_i, l_i, merge=merge)
        e1.record()
        torch.cuda.synchronize()
        per = {name: sum(a.elapsed_time(b) for a, b in spans) for name, spans in marks.items()}
        per["total"] = e0.elapsed_time(e1)
        per["exchange"] = x0.elapsed_time(e1) - per["merge"]
        return per, out_r

    one_pass()                                             # warm-up (NCCL channels, workspace growth)
    dist.barrier()
    torch.cuda.synchronize()
    per, out_r = one_pass()
    vec = torch.tensor([per["total"], per["stats_allreduce"], per["exchange"], per["merge"], per["akl_attention"],
                        per["akl_kv_tile_stats"] + per["akl_kv_means"] + per["akl_kv_scales"] + per["akl_kv_transform"]
                        + per["akl_quantize_q"]], device=dev, dtype=torch.float64)
    dist.all_reduce(vec, op=dist.ReduceOp.MAX)
    fl4 = flops(P4, T4, Hq4)
    sent = (world - 1) / world * (T4 * Hq4 * D * 2 + T4 * Hq4 * 4)
    result.update({
        "c4": f"one request, 32:4, {P4} cached + {T4} new tokens, KV axis cut in {world} at multiples of 1024",
        "c4_ms": float(vec[0]), "c4_tflops": fl4 / float(vec[0]) / 1e9,
        "stats_allreduce_ms": float(vec[1]), "exchange_ms": float(vec[2]), "merge_ms": float(vec[3]),
        "attention_ms": float(vec[4]), "preprocessing_ms": float(vec[5]),
        "exchange_bytes_sent_per_rank": int(sent),
        "exchange_gbs_per_rank": sent / max(float(vec[2]), 1e-9) / 1e6,
        "finite": bool(torch.isfinite(out_r).all()), "status": ws4.status(),
        "timing": "CUDA events on each rank's stream, max over ranks, second pass"})
    return result


def K_load():
    from attn_kernel_lab_b200 import kernel as K_

    return K_.load()


# --------------------------------------------------------------------------------------
# reference legs (test infrastructure: oracle/_ref and oracle/)
# --------------------------------------------------------------------------------------
C1 = {"T": 64, "N": 320, "prefix": 256, "pool": 4096}
C1_SAMPLE = ("configuration 1 exactly: one request, 256 cached + 64 new tokens, 24:4 heads, D 256, BF16 pool of "
             "4096 slots behind a seeded permutation, N(0,1) with 2 % of channels x16, sm_scale 1/16")


def c1_inputs(torch, syn):
    case = {"T": C1["T"], "N": C1["N"], "H": HQ, "KVH": HKV}
    seed = syn.object_seed(1)
    q = syn.outlier_normal((case["T"], HQ, D), seed).to(torch.bfloat16)
    k = syn.outlier_normal((case["N"], HKV, D), seed + 1).to(torch.bfloat16)
    v = syn.outlier_normal((case["N"], HKV, D), seed + 2).to(torch.bfloat16)
    g = torch.Generator().manual_seed(seed + 3)
    idx = torch.randperm(C1["pool"], generator=g)[:C1["N"]].to(torch.int64)
    k_pool = (torch.rand((C1["pool"], HKV, D), generator=g) * 2 - 1).to(torch.bfloat16)
    v_pool = (torch.rand((C1["pool"], HKV, D), generator=g) * 2 - 1).to(torch.bfloat16)
    k_pool[idx] = k
    v_pool[idx] = v
    return q, k_pool, v_pool, idx


def reference_modules():
    """The unmodified reference from oracle/_ref, or None."""
    if not (REF_DIR / "attn_kernel_lab" / "oracle_a.py").exists():
        return None
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    from attn_kernel_lab import oracle_a, quant   # noqa: PLC0415

    return oracle_a, quant


def cpu_reference_c1(repeats: int = 5):
    """Median seconds of the reference's CPU oracle on configuration 1: its shipped INT8 oracle and
    the FP8-QK composition.  Falls back to the oracle port when oracle/_ref is absent."""
    import torch

    from attn_kernel_lab_b200 import synthetic as syn

    q, k_pool, v_pool, idx = c1_inputs(torch, syn)
    rows = idx.long()
    mods = reference_modules()
    fl = flops(C1["prefix"], C1["T"])
    out = {"cores": os.cpu_count(), "torch_threads": torch.get_num_threads(), "sample": C1_SAMPLE,
           "flops": fl, "repeats": repeats}
    try:
        out["cpu_model"] = next(l.split(":", 1)[1].strip() for l in open("/proc/cpuinfo") if l.startswith("model name"))
    except Exception:  # noqa: BLE001
        out["cpu_model"] = None

    def median_time(fn):
        fn()
        ts = []
        for _ in range(repeats):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return statistics.median(ts)

    if mods is not None:
        oracle_a, quant = mods

        def int8_oracle():
            return oracle_a.reference(q, k_pool[rows], v_pool[rows], C1["prefix"], sm_scale=SM_SCALE, return_lse=True)

        def fp8_composition():
            ws = quant.FP8PrefillWorkspace(torch.device("cpu"))
            kvd = quant.gather_quantize_kv(ws, k_pool, v_pool, rows, need_vt8=True, need_vb16=False,
                                           center_k=True, qk_i8=False, rotate=True)
            q8, qscale, mpad = quant.quantize_q(ws, q, SM_SCALE, qk_i8=False, rotate=True)
            nt = kvd["ntmax"]
            ksum = ws.get("ksum", (HKV, D), torch.float32)
            vst = ws.get("vscale_t", (HKV, nt), torch.float32)
            qp = oracle_a.QPack(q8=q8.view(torch.float8_e4m3fn), qscale=qscale, mpad=mpad)
            kvp = oracle_a.KVPack(k8=kvd["k8"].view(torch.float8_e4m3fn), kscale=kvd["kscale"],
                                  kmean=ksum / C1["N"], vt8=kvd["vt8"].view(HKV, nt, D, quant.BLK).view(torch.float8_e4m3fn),
                                  vst_scaled=vst, vscale=kvd["vscale"], vlog2r=kvd["vlog2r"], vinvr=kvd["vinvr"],
                                  vmean=kvd["vmean"], n=C1["N"])
            return oracle_a.attention(qp, kvp, C1["prefix"], C1["T"], group=HQ // HKV, return_lse=True)

        out["kind"] = "reference"
        out["seconds_int8_oracle"] = median_time(int8_oracle)
        out["seconds_fp8_composition"] = median_time(fp8_composition)
        out["seconds"] = out["seconds_fp8_composition"] if not QK_I8 else out["seconds_int8_oracle"]
    else:
        sys.path.insert(0, str(ROOT / "oracle"))
        import akl_oracle as oracle

        qf, kf, vf = q.float().numpy(), k_pool[rows].float().numpy(), v_pool[rows].float().numpy()
        out["kind"] = "port"
        out["seconds"] = median_time(lambda: oracle.reference(qf, kf, vf, C1["prefix"], sm_scale=SM_SCALE, qk_i8=QK_I8))
    out["value"] = fl / out["seconds"] / 1e12
    out["unit"] = "TF/s"
    return out


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    reps = max(args.steps, 1)
    res = cpu_reference_c1(repeats=min(max(reps, 5), 20))
    value = res["value"]
    line = {
        "impl": "reference", "metric": "inclusive_tflops", "value": value, "unit": "TF/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["seconds"] * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f64 oracle over int8/fp8 operands", "data": "synthetic",
        "tokens_per_s": C1["T"] / res["seconds"],
        "config": {"workload": "c1_cpu_oracle", "sample": C1_SAMPLE, "q_heads": HQ, "kv_heads": HKV, "head_dim": D,
                   "note": "the reference's CPU oracle is a Python loop over (head, row); the main workload "
                           "(about 5 M iterations per request-layer) is out of its reach, so its own "
                           "CPU-runnable configuration is timed instead"},
        "cpu_baseline": {k: res[k] for k in res},
        "e2e": {"value": value, "unit": "TF/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def gpu_reference_leg(torch, wl, dev):
    """The reference's own operator on the same box: its mma.sync kernel built for sm_100a (prebuilt
    under oracle/_ref/torch_ext), through its public `ops.prefill_extend`, on request 0 of layer 0."""
    ext_dir = REF_DIR / "torch_ext"
    if reference_modules() is None or not ext_dir.exists():
        return {"unavailable": "oracle/_ref holds no prebuilt reference extension"}
    try:
        import importlib.util

        from attn_kernel_lab import kernel as ref_kernel   # noqa: PLC0415
        from attn_kernel_lab import ops as ref_ops          # noqa: PLC0415

        # the reference's loader would rebuild its extension (a minute and more of compile time) because
        # the build directory moved with the working tree; hand it its own prebuilt module instead --
        # built from its own source with its own flags by oracle/build_ref.py -- through the cache
        # its `load()` consults first
        so = next((ext_dir / "attn_kernel_lab_fp8_prefill").glob("*.so"), None)
        if so is None:
            return {"unavailable": "no prebuilt reference extension under oracle/_ref/torch_ext"}
        spec = importlib.util.spec_from_file_location("attn_kernel_lab_fp8_prefill", so)
        ext = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ext)
        ref_kernel._ext, ref_kernel._loaded_from = ext, "jit"
        r = wl["reqs"][0]
        q = wl["q_all"][0][r["row0"]:r["row0"] + r["T"]]
        kp, vp = wl["k_pools"][0], wl["v_pools"][0]
        idx = r["idx"].long()
        t0 = time.perf_counter()
        ref_out = ref_ops.prefill_extend(q, kp, vp, idx, r["prefix"], sm_scale=SM_SCALE, qk_i8=QK_I8)
        torch.cuda.synchronize()
        first_call_s = time.perf_counter() - t0
        ms = device_time(torch, lambda: ref_ops.prefill_extend(q, kp, vp, idx, r["prefix"], sm_scale=SM_SCALE,
                                                               qk_i8=QK_I8), reps=5, warm=1)
        ours = wl["out_all"][0][r["row0"]:r["row0"] + r["T"]].float()
        d = (ours - ref_out.float()).reshape(-1, D)
        rel = d.norm(dim=1) / ref_out.float().reshape(-1, D).norm(dim=1).clamp_min(1e-30)
        same_rows = float((d == 0).all(dim=1).float().mean())
        same_elems = float((d == 0).float().mean())
        fl = flops(r["prefix"], r["T"])
        return {"kernel": "the reference's fp8_prefill_attn (mma.sync) compiled for sm_100a, inclusive of its "
                          "tensor-library preprocessing", "request": {"prefix": r["prefix"], "T": r["T"]},
                "ms_inclusive": ms, "tflops_inclusive": fl / ms / 1e9, "first_call_s": first_call_s,
                "rowrel_median_vs_this_library": float(rel.median()), "rowrel_max_vs_this_library": float(rel.max()),
                "bit_identical_rows_vs_this_library": same_rows, "bit_identical_elements_vs_this_library": same_elems}
    except Exception as exc:  # noqa: BLE001 - reported, never fatal for the bench line
        return {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}


# --------------------------------------------------------------------------------------
def main():
    global LAYERS, REQUESTS, QK_I8
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=LAYERS,
                    help="pool pairs resident (default: the full 16-layer workload; fewer only for profiling captures)")
    ap.add_argument("--requests", type=int, default=REQUESTS,
                    help="requests per GPU (default 8; fewer only for profiling captures)")
    ap.add_argument("--lanes", type=int, default=2,
                    help="batch workspaces / streams the layers alternate over")
    ap.add_argument("--qk", default="fp8", choices=["fp8", "int8"],
                    help="QK operand type: fp8 (the measured configuration) or int8 (the reference's default mode)")
    ap.add_argument("--launch", default="graph", choices=["graph", "eager"],
                    help="timed steps replay one captured CUDA graph of the step (default) or enqueue eagerly")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-c5", action="store_true")
    ap.add_argument("--no-gpu-reference", action="store_true")
    ap.add_argument("--no-multi", action="store_true", help="skip the strong-scaling and KV-split legs at N > 1")
    args = ap.parse_args()
    LAYERS, REQUESTS, QK_I8 = args.layers, args.requests, args.qk == "int8"
    if args.impl == "reference":
        # launchers such as torchrun pin OMP_NUM_THREADS=1; the CPU leg is meant to use every core
        for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
            os.environ[var] = str(os.cpu_count() or 1)
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    import attn_kernel_lab_b200 as pkg
    from attn_kernel_lab_b200 import kernel as K
    from attn_kernel_lab_b200 import synthetic as syn

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path "
                         "(use --impl reference for the CPU oracle leg)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # a rank that failed inside a leg must not hold the others for the default ten minutes
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=240))
    pkg.load()
    warmup = max(args.warmup, 3)

    wl = build_workload(torch, syn, dev, rank)
    stepper = Stepper(torch, pkg, wl, dev, args.lanes)
    for _ in range(warmup):
        stepper()
    torch.cuda.synchronize()
    step = stepper
    if args.launch == "graph":
        # one step (16 batched calls on capacity-reserved workspaces and caller-owned outputs)
        # captured once and replayed: the way a serving engine drives this operator, and it takes
        # the host's enqueue jitter out of the multi-rank timing
        step = capture(torch, stepper)
        step()                                   # one untimed replay
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) / 1e3
    if any(s != 0 for s in stepper.status()):
        raise SystemExit("device status word set: a bounded wait ran out; no number reported")
    t = torch.tensor([sec], device=dev, dtype=torch.float64)
    t_min = t.clone()
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(t_min, op=dist.ReduceOp.MIN)
    sec_max = float(t.item())
    per_step = sec_max / args.steps
    per_step_fastest_rank = float(t_min.item()) / args.steps
    total_flops = wl["flops_per_step"] * world
    value = total_flops / per_step / 1e12

    e2e = None
    if not args.no_e2e:
        e2e_sec, h2d_b, d2h_b = time_e2e(torch, pkg, wl, dev, max(1, min(args.steps, 3)), warmup)
        t = torch.tensor([e2e_sec], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_sec = float(t.item())
        e2e = {"value": total_flops / e2e_sec / 1e12, "unit": "TF/s", "h2d_bytes_per_step": h2d_b,
               "d2h_bytes_per_step": d2h_b, "h2d_gbs_achieved": h2d_b / e2e_sec / 1e9,
               "d2h_gbs_achieved": d2h_b / e2e_sec / 1e9, "copies_per_layer": {"h2d": 1, "d2h": 1}, "slots": 3}
        if rank == 0:
            up, down = measure_pinned_copy(torch, dev)
            e2e["pinned_copy_peak_gbs"] = {"h2d_alone": up, "d2h_alone": down}
            e2e["limit"] = ("host link: with both directions busy the step moves "
                            f"{(h2d_b + d2h_b) / 1e9:.1f} GB per step through pinned memory")

    peaks = measured_peaks()
    c5 = None
    if not args.no_c5 and (LAYERS, REQUESTS) == (16, 8):
        c5 = c5_serving(torch, dist, pkg, K, syn, dev, rank, world, peaks)
    strong = kvs = None
    if world > 1 and not args.no_multi:
        strong = strong_c2(torch, dist, pkg, syn, dev, rank, world, wl)
        try:
            kvs = kv_split_leg(torch, dist, pkg, syn, dev, rank, world)
        except Exception as exc:  # noqa: BLE001 - the main line still prints
            kvs = {"error": f"{type(exc).__name__}: {str(exc)[:300]}"}

    roofline = cpu = gpu_ref = None
    if rank == 0:
        fp8_peak = measure_fp8_gemm_peak(torch, dev)
        roofline = phase_rooflines(torch, K, stepper, wl, peaks, fp8_peak)
        # secondary (HBM) roofline of the whole operator: one read of each input, one write of the
        # output, per request-layer (2 N Hkv D 2 + 2 T Hq D 2 + N e_idx bytes), over the inclusive time
        step_bytes = sum(2 * r["N"] * HKV * D * 2 + 2 * r["T"] * HQ * D * 2 + r["N"] * 8 for r in wl["reqs"]) * LAYERS
        roofline["hbm_secondary"] = {"algorithmic_bytes_per_step": step_bytes,
                                     "achieved": step_bytes / per_step / 1e9, "peak": peaks["hbm_gbs"],
                                     "unit": "GB/s", "frac": step_bytes / per_step / 1e9 / peaks["hbm_gbs"]}
        if world == 1 and not args.no_cpu:
            cpu = cpu_reference_c1()
        if world == 1 and not args.no_gpu_reference:
            gpu_ref = gpu_reference_leg(torch, wl, dev)
    if rank == 0:
        line = {
            "metric": "inclusive_tflops", "value": value, "unit": "TF/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": per_step * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 QK, fp8_e4m3 PV" if QK_I8 else "fp8_e4m3", "data": "synthetic",
            "tokens_per_s": wl["tokens_per_step"] * world / per_step,
            "token_layers_per_s": wl["tokens_per_step"] * LAYERS * world / per_step,
            "frac_of_nominal_dense_fp8": value / (NOMINAL_FP8_TFLOPS * world),
            "config": {"workload": "c2_main_24x4" if (LAYERS, REQUESTS) == (16, 8) else "c2_main_24x4_reduced_for_profiling",
                       "requests_per_gpu": REQUESTS, "layers": LAYERS,
                       "extend_tokens": T_EXT, "prefixes": [r["prefix"] for r in wl["reqs"]],
                       "q_heads": HQ, "kv_heads": HKV, "head_dim": D, "pool_slots": POOL_ROWS,
                       "qk": args.qk, "kv_dtype": "bfloat16", "page_size": 1, "partition": f"requests x{world}",
                       "entry": "akl_prefill_extend_batch: one batched call (4 launches) per layer",
                       "lanes_per_gpu": args.lanes,
                       "launch": ("one CUDA graph of the step, replayed" if args.launch == "graph" else "eager"),
                       "l2": "inputs larger than L2 (29.3 GB of pools, 3.2 GB of queries per step)"},
            "e2e": e2e,
            "gpu_launches": KERNELS_PER_BATCH * LAYERS * args.steps * world,
            "ms_per_step_fastest_rank": per_step_fastest_rank * 1e3,
            "clocks": clocks.summary(),
            "roofline": roofline,
            "cpu_baseline": cpu,
            "gpu_reference": gpu_ref,
            "c5_serving": c5,
            "strong_c2": strong,
            "kv_split": kvs,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
