"""The benchmark configurations that are not the bench line, at their full sizes, as parity cases:
the GQA sweep over an FP16 pool (16 ragged requests per head ratio), the long single request split
along the KV axis into 8 parts, and the 256-request serving batch replayed from one CUDA graph.

At these sizes the float64 oracle is applied to sampled row blocks (per-row Q quantisation and
per-head K/V statistics make a block exact on its own), and the rest is held by properties that do
not depend on size: batch == one by one, graph replay == eager, split-and-merge == unsplit,
request-wide statistics bit-identical on every part, determinism."""
import numpy as np
import pytest
import torch

import akl_oracle as O
import cases
import helpers as H

pytestmark = pytest.mark.gpu


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def _place(pool_k, pool_v, rows, k, v):
    pool_k[rows] = k.to(pool_k.device, pool_k.dtype)
    pool_v[rows] = v.to(pool_v.device, pool_v.dtype)


# ------------------------------------------------------------------ GQA sweep, FP16 pool
@pytest.mark.parametrize("hq", [16, 32])
def test_gqa_sweep_fp16_pool_sixteen_ragged_requests(pkg, cuda, hq):
    """16 requests, extend length log-uniform in [1, 4096], prefix uniform in [0, 16384], values
    N(0, 0.5) with per-token norm jitter, one shared FP16 pool with a shuffled page table."""
    lens = cases.c3_lengths(16)
    total = sum(p + t for p, t in lens)
    slots = total + 4096
    perm = torch.randperm(slots, generator=torch.Generator().manual_seed(cases.object_seed(3, hq, 3)))
    kp = torch.zeros(slots, 4, 256, dtype=torch.float16, device=cuda)
    vp = torch.zeros(slots, 4, 256, dtype=torch.float16, device=cuda)
    reqs, at = [], 0
    for i, (p, t) in enumerate(lens):
        n = p + t
        seed = cases.object_seed(3, hq, 10 + i)
        q = cases.jitter_normal((t, hq, 256), seed).to(torch.bfloat16)
        k = cases.jitter_normal((n, 4, 256), seed + 1).to(torch.float16)
        v = cases.jitter_normal((n, 4, 256), seed + 2).to(torch.float16)
        rows = perm[at:at + n]
        at += n
        _place(kp, vp, rows.to(cuda), k, v)
        reqs.append({"q": q.to(cuda), "k_pool": kp, "v_pool": vp, "idx": rows.to(cuda), "prefix": p,
                     "out": torch.empty(t, hq, 256, dtype=torch.bfloat16, device=cuda),
                     "lse_out": torch.empty(t, hq, dtype=torch.float32, device=cuda),
                     "cpu": (q, k, v)})
    max_n, max_t = max(p + t for p, t in lens), max(t for _, t in lens)
    wss = [pkg.plan_workspace(cuda, max_kv_len=max_n, max_q_len=max_t, q_heads=hq, kv_heads=4) for _ in range(4)]
    H.fp8_batch(pkg, reqs, workspace=wss, sm_scale=1 / 16, return_lse=True)
    torch.cuda.synchronize()
    assert all(ws.status() == 0 for ws in wss)
    batch = [(r["out"].clone(), r["lse_out"].clone()) for r in reqs]
    # one by one on a single workspace: the same bytes
    for r, (bo, bl) in zip(reqs, batch):
        o, l = H.fp8_extend(pkg, r["q"], kp, vp, r["idx"], r["prefix"], workspace=wss[0], sm_scale=1 / 16,
                                  return_lse=True)
        assert torch.equal(o, bo) and torch.equal(l, bl)
        assert torch.isfinite(o).all()
    # the oracle on row blocks of eight requests (shortest to longest), four q heads each: one per
    # kv head group, 32 rows apiece -- about a thousand (row, head) vectors
    order = sorted(range(16), key=lambda i: lens[i][0] + lens[i][1])
    g = hq // 4
    checked = 0
    for i in order[::2]:
        p, t = lens[i]
        q, k, v = reqs[i]["cpu"]
        r1 = t
        r0 = max(0, t - 32)
        for head in (0, g + 1, 2 * g + g // 2, hq - 1):
            ref, ref_lse = H.oracle_row_block(q, k, v, p, 1 / 16, head, head // g, r0, r1)
            got = batch[i][0][r0:r1, head].float().cpu().numpy()
            H.assert_block_close(got, batch[i][1][r0:r1, head].cpu().numpy(), ref, ref_lse, f"request {i} ({p}+{t}) head {head}")
            checked += r1 - r0
    assert checked >= 256


# ------------------------------------------------------------------ long request, KV split in 8
def test_long_request_split_in_eight_equals_unsplit(pkg, cuda):
    """prefix 131072 + 8192 new tokens, 32:4, BF16 pool walked in 64-slot runs, a planted attention
    sink on the first four keys.  Eight parts, run one after another on this device."""
    T, P, Hq, KVH, world = 8192, 131072, 32, 4, 8
    N = T + P
    slots = 147456
    q, k = cases.sink_qk(T, N, Hq, KVH, cases.object_seed(4, 0, 0))
    v = torch.randn((N, KVH, 256), generator=torch.Generator().manual_seed(cases.object_seed(4, 0, 2))).to(torch.bfloat16)
    idx = cases.run_page_table(slots, N, 64, cases.object_seed(4, 0, 3))
    kp = torch.zeros(slots, KVH, 256, dtype=torch.bfloat16, device=cuda)
    vp = torch.zeros(slots, KVH, 256, dtype=torch.bfloat16, device=cuda)
    _place(kp, vp, idx.to(cuda), k, v)
    qd, idd = q.to(cuda), idx.to(cuda)

    ws = pkg.plan_workspace(cuda, max_kv_len=N, max_q_len=T, q_heads=Hq, kv_heads=KVH)
    whole, whole_lse = H.fp8_extend(pkg, qd, kp, vp, idd, P, workspace=ws, sm_scale=1 / 16, return_lse=True)
    torch.cuda.synchronize()
    assert ws.status() == 0
    kmean, vmean = ws.view("kmean").clone(), ws.view("vmean").clone()
    k8_whole, v8_whole = ws.k8_logical(N), ws.v8_logical(N)

    merged, mlse, wss, ranges, outs, lses = H.emulated_kv_split(pkg, qd, kp, vp, idd, P, 1 / 16, world)
    assert len(ranges) == world and ranges[-1][1] == N and all(lo % 64 == 0 for lo, _ in ranges)
    for w, (lo, hi) in zip(wss, ranges):
        # request-wide statistics are bit-identical on every part, and so are the bytes it holds
        assert torch.equal(w.view("kmean").view(torch.int32), kmean.view(torch.int32))
        assert torch.equal(w.view("vmean").view(torch.int32), vmean.view(torch.int32))
        assert torch.equal(w.k8_logical(hi - lo)[:, :hi - lo], k8_whole[:, lo:hi])
        assert torch.equal(w.v8_logical(hi - lo)[:, :hi - lo], v8_whole[:, lo:hi])
    # parts that lie wholly in the future of a row contribute nothing to it
    last_lse = lses[-1]
    assert torch.isneginf(last_lse[: max(0, ranges[-1][0] - P)]).all()
    # split-and-merge against the unsplit run.  Every part rounds P against its own running
    # maximum, so the two results differ by the E4M3 rounding noise of P (3 significand bits spread
    # over ~1e5 nearly uniform keys), not by fp32 rounding: percent level, and LSE to 2e-3.
    a, b = merged.float(), whole.float()
    rel = (a - b).flatten(0, 1).norm(dim=1) / b.flatten(0, 1).norm(dim=1).clamp_min(1e-30)
    assert rel.median().item() < 8e-2 and rel.max().item() < 0.25
    assert (mlse - whole_lse).abs().max().item() < 2e-3
    # the oracle on the last rows of one head (they see all 139264 keys): the unsplit operator,
    # and the split operator composed the same way (per-part attention with request-wide
    # statistics, partial outputs rounded to BF16, float64 merge)
    r0, r1, head = T - 32, T, 9
    qp, kvp = H.oracle_block_packs(q, k, v, 1 / 16, head, head // 8, r0, r1)
    ref, ref_lse = O.attention(qp, kvp, P + r0, r1 - r0, 1, return_lse=True)
    H.assert_block_close(whole[r0:r1, head].float().cpu().numpy(), whole_lse[r0:r1, head].cpu().numpy(),
                         ref[:, 0], ref_lse[:, 0], "unsplit")
    parts = [O.attention(qp, kvp, P + r0, r1 - r0, 1, return_lse=True, kv_lo=lo, kv_hi=hi) for lo, hi in ranges]
    for (po, pl), o, l in zip(parts, outs, lses):
        H.assert_block_close(o[r0:r1, head].float().cpu().numpy(), l[r0:r1, head].cpu().numpy(),
                             po[:, 0], pl[:, 0], "one part")
    want_o, want_l = O.merge_splits([O.round_to_bf16(po) for po, _ in parts], [pl for _, pl in parts])
    H.assert_block_close(merged[r0:r1, head].float().cpu().numpy(), mlse[r0:r1, head].cpu().numpy(),
                         want_o[:, 0], want_l[:, 0], "split in 8 and merged")
    # three more q heads (the other kv head groups), rows from the middle of the extend: unsplit and merged
    for head, (r0, r1) in ((1, (T // 2 - 32, T // 2)), (18, (T // 4 - 32, T // 4)), (31, (T - 64, T - 32))):
        qp, kvp = H.oracle_block_packs(q, k, v, 1 / 16, head, head // 8, r0, r1)
        ref, ref_lse = O.attention(qp, kvp, P + r0, r1 - r0, 1, return_lse=True)
        H.assert_block_close(whole[r0:r1, head].float().cpu().numpy(), whole_lse[r0:r1, head].cpu().numpy(),
                             ref[:, 0], ref_lse[:, 0], f"unsplit, head {head}")
        parts = [O.attention(qp, kvp, P + r0, r1 - r0, 1, return_lse=True, kv_lo=lo, kv_hi=hi) for lo, hi in ranges]
        want_o, want_l = O.merge_splits([O.round_to_bf16(po) for po, _ in parts], [pl for _, pl in parts])
        H.assert_block_close(merged[r0:r1, head].float().cpu().numpy(), mlse[r0:r1, head].cpu().numpy(),
                             want_o[:, 0], want_l[:, 0], f"split in 8 and merged, head {head}")


# ------------------------------------------------------------------ serving batch from one graph
def test_serving_batch_of_256_requests_replayed_from_one_graph(pkg, cuda):
    """256 requests, extend lengths geometric (mean 128, at most 512), prefixes uniform in
    [0, 32768], 24:4, outlier channels; capacity-reserved workspaces and caller-owned outputs; the
    whole batch captured once, replayed with new query values."""
    from attn_kernel_lab_b200 import dist as D

    lens = cases.c5_lengths(256)
    Hq, KVH = 24, 4
    total = sum(p + t for p, t in lens)
    slots = total + 1024
    g = torch.Generator(device=cuda).manual_seed(cases.object_seed(5, 0, 1))
    scale = torch.where(torch.rand(256, device=cuda, generator=g) < 0.02, 16.0, 1.0)
    scale[7] = 16.0                                   # at least one outlier channel
    kp = (torch.randn(slots, KVH, 256, device=cuda, generator=g) * scale).to(torch.bfloat16)
    vp = (torch.randn(slots, KVH, 256, device=cuda, generator=g) * scale).to(torch.bfloat16)
    perm = torch.randperm(slots, device=cuda, generator=g)
    q_all = (torch.randn(sum(t for _, t in lens), Hq, 256, device=cuda, generator=g) * scale).to(torch.bfloat16)
    out_all = torch.empty_like(q_all)
    reqs, at, row = [], 0, 0
    for p, t in lens:
        reqs.append({"q": q_all[row:row + t], "k_pool": kp, "v_pool": vp, "idx": perm[at:at + p + t].contiguous(),
                     "prefix": p, "out": out_all[row:row + t]})
        at += p + t
        row += t
    # the native batched entry: one capacity-reserved batch workspace, four launches for all 256 requests
    wss = pkg.plan_batch_workspace(cuda, max_requests=256, max_total_kv_len=total,
                                   max_total_q_len=sum(t for _, t in lens), q_heads=Hq, kv_heads=KVH)
    ptrs = wss.base_ptr()

    H.fp8_batch(pkg, reqs, workspace=wss, sm_scale=1 / 16)            # eager
    torch.cuda.synchronize()
    eager = out_all.clone()
    assert torch.isfinite(eager).all() and wss.status() == 0

    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            H.fp8_batch(pkg, reqs, workspace=wss, sm_scale=1 / 16)
    torch.cuda.current_stream().wait_stream(side)
    out_all.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out_all.view(torch.int16), eager.view(torch.int16)), "replay == eager"
    assert wss.base_ptr() == ptrs, "nothing was reallocated"

    # new query values in the same buffers: the replay follows them
    q_all.copy_((q_all.float() * 0.5).to(torch.bfloat16))
    graph.replay()
    torch.cuda.synchronize()
    replay2 = out_all.clone()
    one = pkg.plan_workspace(cuda, max_kv_len=32768 + 512, max_q_len=512, q_heads=Hq, kv_heads=KVH)
    H.fp8_batch(pkg, reqs, workspace=one, sm_scale=1 / 16)            # request by request, single-request entry
    torch.cuda.synchronize()
    assert torch.equal(out_all.view(torch.int16), replay2.view(torch.int16))
    assert not torch.equal(replay2, eager)

    # the oracle on eight requests from the shortest to the deepest context, four q heads each (one
    # per kv head group), up to 32 rows apiece
    order = sorted(range(256), key=lambda i: lens[i][0] + lens[i][1])
    row0 = np.concatenate([[0], np.cumsum([t for _, t in lens])])
    checked = 0
    for i in [order[j] for j in (0, 40, 80, 120, 160, 200, 240, 255)]:
        p, t = lens[i]
        rows = reqs[i]["idx"]
        q = reqs[i]["q"].cpu()
        k, v = kp[rows].cpu(), vp[rows].cpu()
        r0, r1 = max(0, t - 32), t
        for head in (0, 7, 14, 23):
            ref, ref_lse = H.oracle_row_block(q, k, v, p, 1 / 16, head, head // 6, r0, r1)
            got = replay2[row0[i] + r0:row0[i] + r1, head].float().cpu().numpy()
            rel = H.row_rel(got, ref)
            assert np.median(rel) < 2e-3 and (rel < 9e-3).mean() >= 0.9, (i, p, t, head, float(rel.max()))
            checked += r1 - r0
    assert checked >= 256

    # partition by request over 1/2/4/8 ranks covers every request exactly once
    costs = [cases.attention_flops(Hq, t, p) for p, t in lens]
    for world in (1, 2, 4, 8):
        parts = D.partition_requests(costs, world)
        assert len(parts) == world and sorted(i for part in parts for i in part) == list(range(256))
        loads = [sum(costs[i] for i in part) for part in parts]
        assert max(loads) <= 1.05 * sum(costs) / world + max(costs)
