"""Benchmark of the fused FP8 paged EXTEND/prefill attention path.

    python bench.py --gpus N --steps K --warmup W            # this library, on N B200s
    python bench.py --impl reference --steps K --warmup W    # the CPU oracle port on host cores

Workload (`config.workload` = "c2_main_24x4"): the main D256 GQA 24:4 profile -- per GPU 8
requests, prefix ~ U{1024..8192}, 2048 extend tokens each, BF16 K/V pools of 446 464 slots
addressed through one shuffled page table, 16 layers = 16 distinct pool pairs resident in HBM
(29.3 GB), replayed back to back.  One STEP = all 8 requests through all 16 layers = 128
operator calls.  Values ~ N(0,1) with 2 % of channels x16 (seeded, synthetic).

metric   inclusive TF/s: attention FLOPs 4*Hq*D*T*(prefix + (T+1)/2) per request-layer
         (reference bench/candidate_bench.py:210-212) over ONE span holding everything the
         operator does from BF16 inputs to BF16 output (gather, statistics, transform,
         attention, output write; reference bench/candidate_bench.py:876-898).
value    inputs already resident in HBM, timed with CUDA events on the launch stream,
         max over ranks.
e2e      the same metric through `prefill_extend` with HOST buffers: per request-layer the
         query chunk and the chunk's new K/V rows come from pinned host memory (the K/V rows
         are written into the paged pool, as a serving engine does), and the BF16 output goes
         back to pinned host memory; copies overlap compute on their own streams.
roofline the attention kernel alone against the dense-FP8 tensor peak (measured in this run
         with a library FP8 GEMM; 2x the measured BF16 peak of MEASURED_PEAKS.json and the
         vendor nominal are reported beside it).
cpu_baseline  the CPU oracle (oracle/akl_oracle.py, a port of the reference's PyTorch oracle)
         on a bounded sample of the same workload, all host threads.
With N > 1 each rank runs its own 8-request workload (requests are independent units; no
data-path collective): weak scaling, value = all ranks' FLOPs / slowest rank's time.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import pathlib
import subprocess
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
for _p in (ROOT, ROOT / "tests"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

HQ, HKV, D = 24, 4, 256
POOL_ROWS = 446_464
LAYERS = 16
REQUESTS = 8
QK_I8 = False          # --qk int8 runs the reference's default INT8-QK mode instead of FP8-QK
T_EXT = 2048
SM_SCALE = 1.0 / 16.0
NOMINAL_FP8_TFLOPS = 4500.0
KERNELS_PER_CALL = 4          # tile statistics + Q quantise, means + scales, K/V transform, attention


def flops(prefix: int, t: int) -> float:
    return 4.0 * HQ * D * t * (prefix + (t + 1) / 2.0)


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


# --------------------------------------------------------------------------------------
# workload
# --------------------------------------------------------------------------------------
def build_workload(torch, dev, rank: int):
    """Device-resident pools, page tables and queries of one rank (seeded per object)."""
    import cases

    g = torch.Generator(device=dev)

    def outlier(shape, seed, dtype=torch.bfloat16):
        g.manual_seed(seed)
        x = torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
        mask = torch.rand(D, generator=g, device=dev) < 0.02
        mask[seed % D] = True
        x[..., mask] *= 16.0
        return x.to(dtype)

    cfg = 2 + 100 * rank                                   # distinct values and page tables per rank
    # the request lengths are those of rank 0 on every rank: weak scaling means the same work per GPU
    lens = cases.c2_lengths(REQUESTS, seed=cases.object_seed(2, 0, 4))
    gcpu = torch.Generator().manual_seed(cases.object_seed(cfg, 0, 3))
    table = torch.randperm(POOL_ROWS, generator=gcpu).to(dev)
    k_pools, v_pools = [], []
    for layer in range(LAYERS):                            # chunked fill keeps the fp32 temporary small
        kp = torch.empty((POOL_ROWS, HKV, D), dtype=torch.bfloat16, device=dev)
        vp = torch.empty((POOL_ROWS, HKV, D), dtype=torch.bfloat16, device=dev)
        step = POOL_ROWS // 8
        for c in range(8):
            kp[c * step:(c + 1) * step] = outlier((step, HKV, D), cases.object_seed(cfg, c, 1, layer))
            vp[c * step:(c + 1) * step] = outlier((step, HKV, D), cases.object_seed(cfg, c, 2, layer))
        k_pools.append(kp)
        v_pools.append(vp)
    reqs, off = [], 0
    for i, (prefix, t) in enumerate(lens):
        n = prefix + t
        reqs.append({"prefix": prefix, "T": t, "N": n, "idx": table[off:off + n].contiguous(),
                     "q": [outlier((t, HQ, D), cases.object_seed(cfg, i, 0, layer)) for layer in range(LAYERS)],
                     "out": [torch.empty((t, HQ, D), dtype=torch.bfloat16, device=dev) for _ in range(LAYERS)]})
        off += n
    return {"k_pools": k_pools, "v_pools": v_pools, "reqs": reqs,
            "flops_per_step": sum(flops(r["prefix"], r["T"]) for r in reqs) * LAYERS,
            "tokens_per_step": sum(r["T"] for r in reqs)}


def run_step(pkg, wl, ws):
    """One pass: every request through every layer, results in the caller-owned outputs.
    `ws` is a list of workspaces: the 8 independent requests of a layer go through
    `prefill_extend_batch`, which spreads them over that many streams."""
    for layer in range(LAYERS):
        kp, vp = wl["k_pools"][layer], wl["v_pools"][layer]
        pkg.prefill_extend_batch(
            [{"q": r["q"][layer], "k_pool": kp, "v_pool": vp, "idx": r["idx"], "prefix": r["prefix"],
              "out": r["out"][layer]} for r in wl["reqs"]],
            workspace=ws, sm_scale=SM_SCALE, qk_i8=QK_I8)


def time_attention_kernel(torch, pkg, wl, ws, reps: int = 5):
    """Average device time of the attention kernel over the step's launches (layer 0 of every
    request, CUDA events on the launch stream), and the FLOPs those launches carry."""
    from attn_kernel_lab_b200 import kernel as K, quant

    lib = K.load()
    st = torch.cuda.current_stream().cuda_stream
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total_ms, total_flops, launches = 0.0, 0.0, 0
    kp, vp = wl["k_pools"][0], wl["v_pools"][0]
    for r in wl["reqs"]:
        call = quant.make_call(ws, q=r["q"][0], k_pool=kp, v_pool=vp, idx=r["idx"], out=r["out"][0],
                               q_len=r["T"], kv_len=r["N"], prefix=r["prefix"], q_heads=HQ, kv_heads=HKV,
                               sm_scale=SM_SCALE, qk_i8=QK_I8)
        for fn in ("akl_kv_tile_stats", "akl_quantize_q", "akl_kv_means", "akl_kv_scales", "akl_kv_transform"):
            K.check(getattr(lib, fn)(ctypes.byref(call), st), fn)
        K.check(lib.akl_attention(ctypes.byref(call), st), "akl_attention")        # warm
        e0.record()
        for _ in range(reps):
            K.check(lib.akl_attention(ctypes.byref(call), st), "akl_attention")
        e1.record()
        torch.cuda.synchronize()
        total_ms += e0.elapsed_time(e1) / reps
        total_flops += flops(r["prefix"], r["T"])
        launches += 1
    return total_ms / launches, total_flops / launches


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


def time_e2e(torch, pkg, wl, ws, steps: int, warmup: int):
    """Host buffers in, host buffers out, through the public entry point."""
    dev = wl["k_pools"][0].device
    reqs = wl["reqs"]
    host = []
    for r in reqs:
        host.append({
            "q": torch.randn((r["T"], HQ, D)).to(torch.bfloat16).pin_memory(),
            "k": torch.randn((r["T"], HKV, D)).to(torch.bfloat16).pin_memory(),
            "v": torch.randn((r["T"], HKV, D)).to(torch.bfloat16).pin_memory(),
            "out": torch.empty((r["T"], HQ, D), dtype=torch.bfloat16).pin_memory(),
        })
    slots = [{"q": torch.empty((T_EXT, HQ, D), dtype=torch.bfloat16, device=dev),
              "k": torch.empty((T_EXT, HKV, D), dtype=torch.bfloat16, device=dev),
              "v": torch.empty((T_EXT, HKV, D), dtype=torch.bfloat16, device=dev),
              "out": torch.empty((T_EXT, HQ, D), dtype=torch.bfloat16, device=dev),
              "loaded": torch.cuda.Event(), "computed": torch.cuda.Event(), "drained": torch.cuda.Event()}
             for _ in range(2)]
    h2d, d2h, compute = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
    h2d_bytes = sum(h["q"].nbytes + h["k"].nbytes + h["v"].nbytes for h in host) * LAYERS
    d2h_bytes = sum(h["out"].nbytes for h in host) * LAYERS

    def one_step():
        n = 0
        for layer in range(LAYERS):
            kp, vp = wl["k_pools"][layer], wl["v_pools"][layer]
            for r, h in zip(reqs, host):
                s = slots[n % 2]
                with torch.cuda.stream(h2d):
                    h2d.wait_event(s["computed"])                 # slot inputs free again
                    s["q"][:r["T"]].copy_(h["q"], non_blocking=True)
                    s["k"][:r["T"]].copy_(h["k"], non_blocking=True)
                    s["v"][:r["T"]].copy_(h["v"], non_blocking=True)
                    s["loaded"].record(h2d)
                compute.wait_event(s["loaded"])
                compute.wait_event(s["drained"])                  # slot output copied out
                new_rows = r["idx"][r["prefix"]:]
                kp.index_copy_(0, new_rows, s["k"][:r["T"]])       # the chunk's K/V enter the paged pool
                vp.index_copy_(0, new_rows, s["v"][:r["T"]])
                pkg.prefill_extend(s["q"][:r["T"]], kp, vp, r["idx"], r["prefix"], workspace=ws,
                                   out=s["out"][:r["T"]], sm_scale=SM_SCALE, qk_i8=QK_I8)
                s["computed"].record(compute)
                with torch.cuda.stream(d2h):
                    d2h.wait_event(s["computed"])
                    h["out"].copy_(s["out"][:r["T"]], non_blocking=True)
                    s["drained"].record(d2h)
                n += 1
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
# CPU oracle legs
# --------------------------------------------------------------------------------------
CPU_SAMPLE = ("request 0 of the workload cut to its first 512 extend rows (kv length prefix+512), "
              "24:4 heads, one layer: preprocessing + attention through the float64 oracle port")


def cpu_oracle_sample(repeats: int = 1):
    """Seconds per pass and FLOPs of the bounded CPU sample (oracle port, all host threads)."""
    import numpy as np  # noqa: F401
    import torch

    sys.path.insert(0, str(ROOT / "oracle"))
    import akl_oracle as oracle
    import cases

    prefix = cases.c2_lengths(REQUESTS, seed=cases.object_seed(2, 0, 4))[0][0]
    t = 512
    n = prefix + t
    q = cases.outlier_normal((t, HQ, D), cases.object_seed(2, 0, 0)).to(torch.bfloat16).float().numpy()
    k = cases.outlier_normal((n, HKV, D), cases.object_seed(2, 0, 1)).to(torch.bfloat16).float().numpy()
    v = cases.outlier_normal((n, HKV, D), cases.object_seed(2, 0, 2)).to(torch.bfloat16).float().numpy()
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.reference(q, k, v, prefix, sm_scale=SM_SCALE, qk_i8=QK_I8)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best, flops(prefix, t), t


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    for _ in range(min(args.warmup, 1)):
        cpu_oracle_sample()
    times = []
    fl = tok = 0
    for _ in range(args.steps):
        dt, fl, tok = cpu_oracle_sample()
        times.append(dt)
    sec = sum(times) / len(times)
    value = fl / sec / 1e12
    cores = os.cpu_count()
    line = {
        "impl": "reference", "metric": "inclusive_tflops", "value": value, "unit": "TF/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic", "tokens_per_s": tok / sec,
        "config": {"workload": "c2_main_24x4", "sample": CPU_SAMPLE, "q_heads": HQ, "kv_heads": HKV,
                   "head_dim": D},
        "cpu_baseline": {"value": value, "unit": "TF/s", "cores": cores, "kind": "port", "sample": CPU_SAMPLE},
        "e2e": {"value": value, "unit": "TF/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


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
    ap.add_argument("--streams", type=int, default=4,
                    help="workspaces/streams the independent requests of a layer are spread over")
    ap.add_argument("--qk", default="fp8", choices=["fp8", "int8"],
                    help="QK operand type: fp8 (the measured configuration) or int8 (the reference's default mode)")
    ap.add_argument("--launch", default="graph", choices=["graph", "eager"],
                    help="timed steps replay one captured CUDA graph of the step (default) or enqueue eagerly")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
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

    import __graft_entry__ as entry

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path "
                         "(use --impl reference for the CPU oracle leg)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pkg = entry.package()
    pkg.load()
    warmup = max(args.warmup, 3)

    wl = build_workload(torch, dev, rank)
    max_n = max(r["N"] for r in wl["reqs"])
    ws = [pkg.plan_workspace(dev, max_kv_len=max_n, max_q_len=T_EXT, q_heads=HQ, kv_heads=HKV)
          for _ in range(args.streams)]

    for _ in range(warmup):
        run_step(pkg, wl, ws)
    torch.cuda.synchronize()
    step = lambda: run_step(pkg, wl, ws)
    if args.launch == "graph":
        # one step (128 operator calls on capacity-reserved workspaces and caller-owned outputs)
        # captured once and replayed: the way a serving engine drives this operator, and it takes
        # the host's enqueue jitter out of the multi-rank timing
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                run_step(pkg, wl, ws)
        torch.cuda.current_stream().wait_stream(side)
        step = graph.replay
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
    if any(w.status() != 0 for w in ws):
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

    e2e_value = h2d_b = d2h_b = None
    if not args.no_e2e:
        e2e_sec, h2d_b, d2h_b = time_e2e(torch, pkg, wl, ws[0], max(1, min(args.steps, 3)), warmup)
        t = torch.tensor([e2e_sec], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_value = total_flops / float(t.item()) / 1e12

    roofline = cpu = None
    if rank == 0:
        peaks = measured_peaks()
        attn_ms, attn_flops = time_attention_kernel(torch, pkg, wl, ws[0])
        fp8_peak = measure_fp8_gemm_peak(torch, dev)
        peak = fp8_peak if fp8_peak else 2.0 * peaks["bf16_tflops"]
        achieved = attn_flops / attn_ms / 1e9
        traffic = None
        tpath = ROOT / "profiles" / "attn_sm100_traffic.json"
        if tpath.exists():
            traffic = json.loads(tpath.read_text()).get("dram_bytes_per_launch")
        roofline = {"bound": "tensor", "kernel": "attn_sm100_kernel", "achieved": achieved, "peak": peak,
                    "unit": "TFLOP/s", "frac": achieved / peak, "traffic": traffic,
                    "peak_source": ("measured FP8 E4M3 GEMM 8192^3 in this run (tensor library, burst)"
                                    if fp8_peak else "2 x measured BF16 burst peak (MEASURED_PEAKS.json)"),
                    "frac_of_2x_measured_bf16_burst": achieved / (2.0 * peaks["bf16_tflops"]),
                    "frac_of_2x_measured_bf16_sustained": achieved / (2.0 * peaks["bf16_tflops_sustained"]),
                    "frac_of_nominal_dense_fp8": achieved / NOMINAL_FP8_TFLOPS,
                    "attention_ms_per_launch": attn_ms, "flops_per_launch": attn_flops}
        # secondary (HBM) roofline of the whole operator: one read of each input, one write of the
        # output, per request-layer (2 N Hkv D 2 + 2 T Hq D 2 + N e_idx bytes), over the inclusive time
        step_bytes = sum(2 * r["N"] * HKV * D * 2 + 2 * r["T"] * HQ * D * 2 + r["N"] * 8 for r in wl["reqs"]) * LAYERS
        roofline["hbm_secondary"] = {"algorithmic_bytes_per_step": step_bytes,
                                     "achieved": step_bytes / per_step / 1e9, "peak": peaks["hbm_gbs"],
                                     "unit": "GB/s", "frac": step_bytes / per_step / 1e9 / peaks["hbm_gbs"]}
        if world == 1 and not args.no_cpu:
            dt, fl, _ = cpu_oracle_sample()
            cpu = {"value": fl / dt / 1e12, "unit": "TF/s", "cores": os.cpu_count(), "kind": "port",
                   "sample": CPU_SAMPLE, "seconds": dt}
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
                       "streams_per_gpu": args.streams,
                       "launch": ("one CUDA graph of the step, replayed" if args.launch == "graph" else "eager"),
                       "l2": "inputs larger than L2 (29.3 GB of pools, 3.2 GB of queries per step)"},
            "e2e": ({"value": e2e_value, "unit": "TF/s", "h2d_bytes_per_step": h2d_b, "d2h_bytes_per_step": d2h_b}
                    if e2e_value is not None else None),
            "gpu_launches": KERNELS_PER_CALL * REQUESTS * LAYERS * args.steps * world,
            "ms_per_step_fastest_rank": per_step_fastest_rank * 1e3,
            "clocks": clocks.summary(),
            "roofline": roofline,
            "cpu_baseline": cpu,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
