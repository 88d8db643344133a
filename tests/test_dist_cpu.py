"""Host logic of the multi-GPU forms, on CPU: pure planners, and the KV-axis split
choreography (statistics made global, all-to-all of partial states, merge) run as two `gloo`
ranks with the CUDA phases replaced by an oracle stand-in that fills the same workspace
regions.  What the ranks exchange and in what order is the code under test; the arithmetic
stand-in is the checker."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import akl_oracle as O
import cases


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


# ------------------------------------------------------------------ planners
def test_partition_requests_balances_flops(pkg):
    from attn_kernel_lab_b200 import dist as D

    lens = cases.c5_lengths(64)
    costs = [cases.attention_flops(24, t, p) for p, t in lens]
    for world in (1, 2, 4, 8):
        bins = D.partition_requests(costs, world)
        assert sorted(i for b in bins for i in b) == list(range(64))
        loads = [sum(costs[i] for i in b) for b in bins]
        assert max(loads) <= sum(costs) / world + max(costs)
    assert D.partition_requests([5.0, 1.0, 1.0], 2) == [[0], [1, 2]]
    assert D.partition_requests([], 2) == [[], []]


def test_kv_split_ranges_are_tile_aligned_and_cover(pkg):
    from attn_kernel_lab_b200 import dist as D

    r = D.kv_split_ranges(139264, 8)
    assert r[0] == (0, 17408) and r[-1] == (121856, 139264) and all(lo % 1024 == 0 for lo, _ in r)
    assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
    r = D.kv_split_ranges(2500, 4)
    assert r == [(0, 1024), (1024, 2048), (2048, 2500), (2500, 2500)]
    assert D.row_slices(10, 4) == [(0, 3), (3, 6), (6, 9), (9, 10)]
    assert D.kv_head_slice(32, 4, 1, 2) == ((16, 32), (2, 4))
    assert D.kv_head_slice(24, 4, 3, 4) == ((18, 24), (3, 4))
    with pytest.raises(ValueError):
        D.kv_head_slice(24, 4, 0, 3)


# ------------------------------------------------------------------ two gloo ranks
CASES = {
    # 96 rows divide over two ranks: the partial states themselves are the all-to-all send buffers
    "even_rows": cases._case("split2", 96, 2500, 2404, 16, 4, "scattered", "outlier", 4301),
    # 97 rows do not: the exchange pads them to 98
    "odd_rows": cases._case("split2odd", 97, 2500, 2403, 16, 4, "scattered", "outlier", 4302),
}
CASE = CASES["even_rows"]


class OraclePhases:
    """Stand-in for the native phase entry points: same inputs, same workspace regions
    written, arithmetic by the CPU oracle."""

    def __init__(self, ws, q, k_local, v_local, out, lse, prefix, sm_scale):
        self.ws, self.q, self.k, self.v = ws, q, k_local, v_local
        self.out, self.lse, self.prefix, self.sm_scale = out, lse, prefix, sm_scale

    def __call__(self, name, call):
        ws = self.ws
        n = self.k.shape[0]
        nt = (n + 63) // 64
        if name == "akl_kv_tile_stats":
            for arr, src in ((ws.view("ktsum"), self.k), (ws.view("vtsum"), self.v)):
                for t in range(nt):
                    rows = src[t * 64:(t + 1) * 64]
                    arr[call.tile0_global + t] = torch.from_numpy(O.channel_sums_tiled(rows))
        elif name == "akl_kv_means":
            ntg = call.ntiles_global
            for key, arr in (("kmean", ws.view("ktsum")), ("vmean", ws.view("vtsum"))):
                total = np.zeros((self.k.shape[1], 256), np.float32)
                tiles = arr[:ntg].numpy()
                for s0 in range(0, ntg, 512):
                    slab = np.zeros_like(total)
                    for t in range(s0, min(s0 + 512, ntg)):
                        slab = (slab + tiles[t]).astype(np.float32)
                    total = (total + slab).astype(np.float32)
                ws.view(key).copy_(torch.from_numpy((total / np.float32(call.n_total)).astype(np.float32)))
            pack = O.preprocess_kv(self.k, self.v, kmean=ws.view("kmean").numpy(), vmean=ws.view("vmean").numpy())
            ws.view("vsmax").copy_(torch.from_numpy(pack.vsmax_local))
        elif name == "akl_attention":
            pack = O.preprocess_kv(self.k, self.v, kmean=ws.view("kmean").numpy(),
                                   vmean=ws.view("vmean").numpy(), vsmax_raw=ws.view("vsmax").numpy())
            qp = O.preprocess_q(self.q, self.sm_scale)
            T, H = self.q.shape[0], self.q.shape[1]
            o, l = O.attention(qp, pack, self.prefix - call.kv_pos0, T, H // self.k.shape[1], return_lse=True)
            self.out.copy_(torch.from_numpy(o).to(torch.bfloat16))
            self.lse.copy_(torch.from_numpy(l))
        # akl_kv_scales / akl_kv_transform / akl_quantize_q are folded into the attention stand-in


def _oracle_merge(parts_o, parts_l):
    o, l = O.merge_splits([p.float().numpy() for p in parts_o], [p.numpy() for p in parts_l])
    return torch.from_numpy(o).to(torch.bfloat16), torch.from_numpy(l)


def _rank_main(rank: int, world: int, port: int, result_path: str, case_key: str):
    CASE = CASES[case_key]
    import sys
    import pathlib

    root = pathlib.Path(__file__).resolve().parents[1]
    for p in (root, root / "tests", root / "oracle"):
        sys.path.insert(0, str(p))
    import __graft_entry__ as entry

    pkg = entry.package()
    from attn_kernel_lab_b200 import dist as D
    from attn_kernel_lab_b200 import quant

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        inp = cases.make_inputs(CASE)
        n_total = CASE["N"]
        lo, hi = D.kv_split_ranges(n_total, world)[rank]
        idx_local = inp["idx"][lo:hi]
        k_local = inp["k_pool"][idx_local].float().numpy()
        v_local = inp["v_pool"][idx_local].float().numpy()
        q = inp["q"]
        ws = pkg.FP8PrefillWorkspace(torch.device("cpu"))

        captured = {}
        orig_make_call = quant.make_call

        def spy_make_call(ws_, **kw):               # the stand-in writes the op's own out / lse
            captured["out"], captured["lse"] = kw["out"], kw["lse_out"]
            return orig_make_call(ws_, **kw)

        quant.make_call = spy_make_call

        class Lazy:
            def __call__(self, name, call):
                OraclePhases(ws, q.float().numpy(), k_local, v_local, captured["out"], captured["lse"],
                             CASE["prefix"], CASE["sm_scale"])(name, call)

        out, lse, (rlo, rhi) = D.prefill_extend_kv_split(
            ws, q, inp["k_pool"], inp["v_pool"], idx_local, CASE["prefix"], n_total=n_total, kv_lo=lo,
            sm_scale=CASE["sm_scale"], phases=Lazy(), merge=_oracle_merge)
        torch.save({"out": out, "lse": lse, "rows": (rlo, rhi), "kmean": ws.view("kmean").clone(),
                    "vmean": ws.view("vmean").clone(), "vsmax": ws.view("vsmax").clone()},
                   f"{result_path}.{rank}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case_key", ["even_rows", "odd_rows"])
def test_kv_split_choreography_two_gloo_ranks(pkg, tmp_path, case_key):
    CASE = CASES[case_key]
    world = 2
    port = _free_port()
    path = str(tmp_path / "res")
    mp.spawn(_rank_main, args=(world, port, path, case_key), nprocs=world, join=True)
    parts = [torch.load(f"{path}.{r}") for r in range(world)]

    # single-process answer: request-wide statistics, per-split operator, float64 merge
    inp = cases.make_inputs(CASE)
    rows = inp["idx"]
    q = inp["q"].float().numpy()
    k = inp["k_pool"][rows].float().numpy()
    v = inp["v_pool"][rows].float().numpy()
    whole = O.preprocess_kv(k, v)
    for p in parts:                                  # disjoint-support SUM all-reduce moved every value unchanged
        assert np.array_equal(p["kmean"].numpy().view(np.uint32), whole.kmean.view(np.uint32))
        assert np.array_equal(p["vmean"].numpy().view(np.uint32), whole.vmean.view(np.uint32))
        assert np.array_equal(p["vsmax"].numpy(), whole.vsmax_local)
    qp = O.preprocess_q(q, CASE["sm_scale"])
    outs, lses = [], []
    from attn_kernel_lab_b200 import dist as D

    for lo, hi in D.kv_split_ranges(CASE["N"], world):
        o, l = O.attention(qp, whole, CASE["prefix"], CASE["T"], 4, return_lse=True, kv_lo=lo, kv_hi=hi)
        outs.append(O.round_to_bf16(o))
        lses.append(l)
    want_o, want_l = O.merge_splits(outs, lses)
    got_o = np.zeros_like(want_o)
    got_l = np.zeros_like(want_l)
    covered = 0
    for p in parts:
        lo, hi = p["rows"]
        got_o[lo:hi] = p["out"].float().numpy()
        got_l[lo:hi] = p["lse"].numpy()
        covered += hi - lo
    assert covered == CASE["T"]
    assert np.array_equal(got_o, want_o)
    assert np.allclose(got_l, want_l, atol=1e-6)
