"""KV-axis split of one request on real GPUs (one process per GPU, NCCL): request-wide
statistics through the disjoint-support SUM and the MAX all-reduce, per-rank attention with
global causal positions, all-to-all of the partial states and the merge kernel.  Checked against
the per-split oracle with request-wide statistics and the float64 merge: a small case on two GPUs,
and the long-context configuration (131072 cached + 8192 new tokens, 32:4) on every GPU of the
machine.  Skipped on a single GPU; the same choreography runs on every machine as two gloo ranks in
tests/test_dist_cpu.py and as consecutive per-rank calls on one GPU in tests/test_gpu_configs.py."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

import akl_oracle as O
import cases
import helpers as H

pytestmark = pytest.mark.gpu
CASE = cases._case("split_nccl", 160, 5000, 4840, 32, 4, "scattered", "outlier", 5101)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, path: str):
    import pathlib
    import sys

    root = pathlib.Path(__file__).resolve().parents[1]
    for p in (root, root / "tests", root / "oracle"):
        sys.path.insert(0, str(p))
    import torch.distributed as dist

    import __graft_entry__ as entry

    pkg = entry.package()
    from attn_kernel_lab_b200 import dist as D

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        inp = cases.make_inputs(CASE)
        lo, hi = D.kv_split_ranges(CASE["N"], world)[rank]
        q, kp, vp = inp["q"].to(dev), inp["k_pool"].to(dev), inp["v_pool"].to(dev)
        idx_local = inp["idx"][lo:hi].contiguous().to(dev)
        ws = pkg.FP8PrefillWorkspace(dev)
        out, lse, (rlo, rhi) = D.prefill_extend_kv_split(
            ws, q, kp, vp, idx_local, CASE["prefix"], n_total=CASE["N"], kv_lo=lo, sm_scale=CASE["sm_scale"])
        torch.cuda.synchronize()
        assert ws.status() == 0
        torch.save({"out": out.cpu(), "lse": lse.cpu(), "rows": (rlo, rhi),
                    "kmean": ws.view("kmean").cpu(), "vmean": ws.view("vmean").cpu()}, f"{path}.{rank}")
    finally:
        dist.destroy_process_group()


def test_kv_split_on_two_gpus_over_nccl(pkg, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world, port, path = 2, _free_port(), str(tmp_path / "res")
    mp.spawn(_rank_main, args=(world, port, path), nprocs=world, join=True)
    parts = [torch.load(f"{path}.{r}") for r in range(world)]
    inp = cases.make_inputs(CASE)
    qf, kf, vf = H.gathered(inp)
    whole = O.preprocess_kv(kf, vf)
    for p in parts:          # the all-reduces left bit-identical request-wide means on both ranks
        assert np.array_equal(p["kmean"].numpy().view(np.uint32), whole.kmean.view(np.uint32))
        assert np.array_equal(p["vmean"].numpy().view(np.uint32), whole.vmean.view(np.uint32))
    from attn_kernel_lab_b200 import dist as D

    qp = O.preprocess_q(qf, CASE["sm_scale"])
    refs = [O.attention(qp, whole, CASE["prefix"], CASE["T"], 8, return_lse=True, kv_lo=lo, kv_hi=hi)
            for lo, hi in D.kv_split_ranges(CASE["N"], world)]
    want_o, want_l = O.merge_splits([O.round_to_bf16(r[0]) for r in refs], [r[1] for r in refs])
    got_o = np.zeros_like(want_o)
    got_l = np.zeros_like(want_l)
    covered = 0
    for p in parts:
        lo, hi = p["rows"]
        got_o[lo:hi] = p["out"].float().numpy()
        got_l[lo:hi] = p["lse"].numpy()
        covered += hi - lo
    assert covered == CASE["T"]
    assert np.abs(got_l - want_l).max() < 5e-3
    rel = H.row_rel(got_o, want_o)
    assert np.median(rel) < 2e-3 and (rel < 9e-3).mean() > 0.95


# ------------------------------------------------------------------ the long-context configuration
LONG_T, LONG_P, LONG_HQ, LONG_KVH, LONG_SLOTS = 8192, 131072, 32, 4, 147456
BLOCK = (LONG_T - 32, LONG_T, 9)          # rows and q head checked against the oracle


def _long_inputs():
    n = LONG_T + LONG_P
    q, k = cases.sink_qk(LONG_T, n, LONG_HQ, LONG_KVH, cases.object_seed(4, 0, 0))
    v = torch.randn((n, LONG_KVH, 256), generator=torch.Generator().manual_seed(cases.object_seed(4, 0, 2))).to(torch.bfloat16)
    idx = cases.run_page_table(LONG_SLOTS, n, 64, cases.object_seed(4, 0, 3))
    return q, k, v, idx


def _long_rank_main(rank: int, world: int, port: int, path: str):
    import pathlib
    import sys

    root = pathlib.Path(__file__).resolve().parents[1]
    for p in (root, root / "tests", root / "oracle"):
        sys.path.insert(0, str(p))
    import torch.distributed as dist

    import __graft_entry__ as entry

    pkg = entry.package()
    from attn_kernel_lab_b200 import dist as D

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        q, k, v, idx = _long_inputs()
        n = LONG_T + LONG_P
        lo, hi = D.kv_split_ranges(n, world)[rank]
        # a rank holds only the pool rows of its own slice of the page table
        kp = torch.zeros(LONG_SLOTS, LONG_KVH, 256, dtype=torch.bfloat16, device=dev)
        vp = torch.zeros(LONG_SLOTS, LONG_KVH, 256, dtype=torch.bfloat16, device=dev)
        mine = idx[lo:hi].to(dev)
        kp[mine] = k[lo:hi].to(dev)
        vp[mine] = v[lo:hi].to(dev)
        ws = pkg.FP8PrefillWorkspace(dev)
        out, lse, (rlo, rhi) = D.prefill_extend_kv_split(
            ws, q.to(dev), kp, vp, mine.contiguous(), LONG_P, n_total=n, kv_lo=lo, sm_scale=1 / 16)
        torch.cuda.synchronize()
        assert ws.status() == 0
        r0, r1, head = BLOCK
        a, b = max(r0, rlo), min(r1, rhi)
        keep = {"rows": (rlo, rhi), "kmean": ws.view("kmean").cpu(), "vmean": ws.view("vmean").cpu(),
                "block_rows": (a, b)}
        if a < b:
            keep["block_out"] = out[a - rlo:b - rlo, head].float().cpu()
            keep["block_lse"] = lse[a - rlo:b - rlo, head].cpu()
        keep["finite"] = bool(torch.isfinite(out).all())
        torch.save(keep, f"{path}.{rank}")
    finally:
        dist.destroy_process_group()


def test_long_context_kv_split_over_nccl_on_every_gpu(pkg, tmp_path):
    world = torch.cuda.device_count()
    if world < 2:
        pytest.skip("needs at least two GPUs")
    world = min(world, 8)
    port, path = _free_port(), str(tmp_path / "long")
    mp.spawn(_long_rank_main, args=(world, port, path), nprocs=world, join=True)
    parts = [torch.load(f"{path}.{r}") for r in range(world)]
    assert all(p["finite"] for p in parts)
    assert sum(p["rows"][1] - p["rows"][0] for p in parts) == LONG_T
    for p in parts[1:]:           # the all-reduces left bit-identical request-wide means everywhere
        assert torch.equal(p["kmean"].view(torch.int32), parts[0]["kmean"].view(torch.int32))
        assert torch.equal(p["vmean"].view(torch.int32), parts[0]["vmean"].view(torch.int32))
    from attn_kernel_lab_b200 import dist as D

    q, k, v, _ = _long_inputs()
    r0, r1, head = BLOCK
    qp, kvp = H.oracle_block_packs(q, k, v, 1 / 16, head, head // 8, r0, r1)
    assert np.array_equal(parts[0]["kmean"].numpy()[head // 8].view(np.uint32), kvp.kmean[0].view(np.uint32))
    refs = [O.attention(qp, kvp, LONG_P + r0, r1 - r0, 1, return_lse=True, kv_lo=lo, kv_hi=hi)
            for lo, hi in D.kv_split_ranges(LONG_T + LONG_P, world)]
    want_o, want_l = O.merge_splits([O.round_to_bf16(o) for o, _ in refs], [l for _, l in refs])
    got_o = np.zeros((r1 - r0, 256), np.float32)
    got_l = np.zeros(r1 - r0, np.float32)
    seen = 0
    for p in parts:
        a, b = p["block_rows"]
        if a < b:
            got_o[a - r0:b - r0] = p["block_out"].numpy()
            got_l[a - r0:b - r0] = p["block_lse"].numpy()
            seen += b - a
    assert seen == r1 - r0
    H.assert_block_close(got_o, got_l, want_o[:, 0], want_l[:, 0], f"split over {world} GPUs")
