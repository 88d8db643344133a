"""KV-axis split of one request on two real GPUs (one process per GPU, NCCL): request-wide
statistics through the disjoint-support SUM and the MAX all-reduce, per-rank attention with
global causal positions, all-to-all of the partial states and the merge kernel.  Checked against
the per-split oracle with request-wide statistics and the float64 merge.  Skipped on a single GPU;
the same choreography runs on every machine as two gloo ranks in tests/test_dist_cpu.py."""
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
