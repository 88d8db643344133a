"""The native batched entry (`akl_prefill_extend_batch`, through `prefill_extend_batch` with an
`FP8PrefillBatchWorkspace`) against the single-request operator: every request's BF16 output and
base-2 LSE bit-equal to `prefill_extend`, in both QK modes, for ragged batches, mixed pools, repeated
use of one workspace, and a CUDA graph replayed after lengths, request count and tensors changed."""
import numpy as np
import pytest
import torch

import cases
import helpers as H

pytestmark = pytest.mark.gpu


def bits(a):
    return a.contiguous().view(torch.int16 if a.dtype == torch.bfloat16 else torch.int32)


def _pool(cuda, slots, KVH, seed, dtype=torch.bfloat16):
    g = torch.Generator(device=cuda).manual_seed(seed)
    scale = torch.where(torch.rand(256, device=cuda, generator=g) < 0.02, 16.0, 1.0)
    scale[seed % 256] = 16.0
    kp = (torch.randn(slots, KVH, 256, device=cuda, generator=g) * scale).to(dtype)
    vp = (torch.randn(slots, KVH, 256, device=cuda, generator=g) * scale).to(dtype)
    return kp, vp, scale, g


def _requests(cuda, lens, Hq, kp, vp, scale, g, idx_dtype=torch.int64, lse=False):
    slots = kp.shape[0]
    perm = torch.randperm(slots, device=cuda, generator=g)
    reqs, at = [], 0
    for p, t in lens:
        q = (torch.randn(t, Hq, 256, device=cuda, generator=g) * scale).to(torch.bfloat16)
        r = {"q": q, "k_pool": kp, "v_pool": vp, "idx": perm[at:at + p + t].to(idx_dtype).contiguous(),
             "prefix": p, "out": torch.full_like(q, float("nan"))}
        if lse:
            r["lse_out"] = torch.full((t, Hq), float("nan"), dtype=torch.float32, device=cuda)
        reqs.append(r)
        at += p + t
    return reqs


def _one_by_one(pkg, reqs, qk_i8, lse=False, **kw):
    ws = pkg.FP8PrefillWorkspace(reqs[0]["q"].device)
    outs = []
    for r in reqs:
        res = pkg.prefill_extend(r["q"], r["k_pool"], r["v_pool"], r["idx"], r["prefix"], workspace=ws,
                                 sm_scale=1 / 16, qk_i8=qk_i8, return_lse=lse, **kw)
        outs.append(tuple(x.clone() for x in res) if lse else res.clone())
    torch.cuda.synchronize()
    assert ws.status() == 0
    return outs


LENS = [(300, 130), (0, 5), (1000, 256), (64, 64), (7, 1), (511, 129), (2047, 1), (129, 300)]


@pytest.mark.parametrize("qk_i8", [False, True], ids=["fp8qk", "int8qk"])
def test_native_batch_is_bit_equal_to_the_single_request_operator(pkg, cuda, qk_i8):
    Hq, KVH = 24, 4
    total = sum(p + t for p, t in LENS)
    kp, vp, scale, g = _pool(cuda, total + 333, KVH, 501)
    reqs = _requests(cuda, LENS, Hq, kp, vp, scale, g, lse=True)
    ref = _one_by_one(pkg, reqs, qk_i8, lse=True)
    bws = pkg.plan_batch_workspace(cuda, max_requests=len(LENS), max_total_kv_len=total,
                                   max_total_q_len=sum(t for _, t in LENS), q_heads=Hq, kv_heads=KVH)
    res = pkg.prefill_extend_batch(reqs, workspace=bws, sm_scale=1 / 16, qk_i8=qk_i8, return_lse=True)
    torch.cuda.synchronize()
    assert bws.status() == 0
    for i, ((o, l), (ro, rl)) in enumerate(zip(res, ref)):
        assert o.data_ptr() == reqs[i]["out"].data_ptr() and l.data_ptr() == reqs[i]["lse_out"].data_ptr()
        assert torch.equal(bits(o), bits(ro)), f"request {i} {LENS[i]}: output bits differ"
        assert torch.equal(bits(l), bits(rl)), f"request {i} {LENS[i]}: lse bits differ"
    # the same workspace again, the batch in another order and without caller-owned outputs
    order = [3, 0, 7, 1]
    again = pkg.prefill_extend_batch([{k: v for k, v in reqs[i].items() if k not in ("out", "lse_out")} for i in order],
                                     workspace=bws, sm_scale=1 / 16, qk_i8=qk_i8)
    torch.cuda.synchronize()
    for i, o in zip(order, again):
        assert torch.equal(bits(o), bits(ref[i][0]))


def test_native_batch_variants_fp16_pool_int32_index_modes_and_mixed_pools(pkg, cuda):
    Hq, KVH = 16, 4
    lens = [(100, 37), (0, 128), (450, 200)]
    total = sum(p + t for p, t in lens)
    kp, vp, scale, g = _pool(cuda, total + 100, KVH, 502, dtype=torch.float16)
    reqs = _requests(cuda, lens, Hq, kp, vp, scale, g, idx_dtype=torch.int32)
    bws = pkg.plan_batch_workspace(cuda, max_requests=4, max_total_kv_len=2 * total, max_total_q_len=1024,
                                   q_heads=Hq, kv_heads=KVH, capability=pkg.GENERALIZATION_CAPABILITY)
    for kw in (dict(), dict(rotate=False), dict(center_k=False)):
        ref = _one_by_one(pkg, reqs, False, capability=pkg.GENERALIZATION_CAPABILITY, **kw)
        res = H.fp8_batch(pkg, reqs, workspace=bws, sm_scale=1 / 16, capability=pkg.GENERALIZATION_CAPABILITY, **kw)
        torch.cuda.synchronize()
        for i, (o, ro) in enumerate(zip(res, ref)):
            assert torch.equal(bits(o), bits(ro)), (kw, i)
    # a second pool of another dtype and index width in the same batch: grouped, still request by request
    kp2, vp2, scale2, g2 = _pool(cuda, 700, KVH, 503, dtype=torch.bfloat16)
    more = _requests(cuda, [(200, 60), (10, 90)], Hq, kp2, vp2, scale2, g2, idx_dtype=torch.int64)
    mixed = [reqs[0], more[0], reqs[2], more[1]]
    ref = _one_by_one(pkg, mixed, False, capability=pkg.GENERALIZATION_CAPABILITY)
    res = H.fp8_batch(pkg, mixed, workspace=bws, sm_scale=1 / 16, capability=pkg.GENERALIZATION_CAPABILITY)
    torch.cuda.synchronize()
    assert bws.status() == 0
    for i, (o, ro) in enumerate(zip(res, ref)):
        assert torch.equal(bits(o), bits(ro)), i
    with pytest.raises(pkg.WorkspaceCapacityError):       # five requests of one group, capacity four
        H.fp8_batch(pkg, reqs + reqs[:2], workspace=bws, sm_scale=1 / 16, capability=pkg.GENERALIZATION_CAPABILITY)


def test_graph_of_the_native_batch_follows_a_replanned_table(pkg, cuda):
    """One captured graph (table copy + four launches); between replays the host table is
    rewritten for other lengths, another request count and other tensors.  No re-capture."""
    Hq, KVH = 24, 4
    kp, vp, scale, g = _pool(cuda, 9000, KVH, 504)
    first = _requests(cuda, [(700, 130), (50, 50), (1500, 300), (0, 64)], Hq, kp, vp, scale, g)
    second = _requests(cuda, [(1200, 400), (3, 2), (800, 128)], Hq, kp, vp, scale, g)
    bws = pkg.plan_batch_workspace(cuda, max_requests=6, max_total_kv_len=4000, max_total_q_len=1000,
                                   q_heads=Hq, kv_heads=KVH)
    plan = bws.plan(first, sm_scale=1 / 16, qk_i8=False)
    bws.launch(plan)                                   # eager once (loads the module, warms up)
    torch.cuda.synchronize()
    ref_first = _one_by_one(pkg, first, False)
    for r, ro in zip(first, ref_first):
        assert torch.equal(bits(r["out"]), bits(ro))

    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            bws.launch(plan)
    torch.cuda.current_stream().wait_stream(side)
    for r in first:
        r["out"].fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    for r, ro in zip(first, ref_first):
        assert torch.equal(bits(r["out"]), bits(ro)), "replay == eager"

    bws.replan(plan, second)                           # host memory only
    graph.replay()
    torch.cuda.synchronize()
    assert bws.status() == 0
    ref_second = _one_by_one(pkg, second, False)
    for r, ro in zip(second, ref_second):
        assert torch.equal(bits(r["out"]), bits(ro)), "replay after replanning"
    with pytest.raises(pkg.WorkspaceCapacityError):
        bws.replan(plan, first + second)


def test_serving_shaped_batch_native_entry_equals_the_stream_batch(pkg, cuda):
    """64 requests drawn like the 256-request serving configuration (extend ~ geometric mean 128
    capped at 512, prefix ~ U{0..32768} scaled down to 0..8192), one native batch."""
    Hq, KVH = 24, 4
    lens = [(p // 4, t) for p, t in cases.c5_lengths(64, seed=cases.object_seed(5, 1, 4))]
    total = sum(p + t for p, t in lens)
    kp, vp, scale, g = _pool(cuda, total + 512, KVH, 505)
    reqs = _requests(cuda, lens, Hq, kp, vp, scale, g)
    bws = pkg.plan_batch_workspace(cuda, max_requests=64, max_total_kv_len=total,
                                   max_total_q_len=sum(t for _, t in lens), q_heads=Hq, kv_heads=KVH)
    H.fp8_batch(pkg, reqs, workspace=bws, sm_scale=1 / 16)
    torch.cuda.synchronize()
    assert bws.status() == 0
    got = [r["out"].clone() for r in reqs]
    ref = _one_by_one(pkg, reqs, False)
    bad = [i for i, (o, ro) in enumerate(zip(got, ref)) if not torch.equal(bits(o), bits(ro))]
    assert not bad, f"requests {bad[:8]} differ from the single-request operator"
    # and one request against the oracle, so that the comparison is not only the CUDA path with itself
    i = max(range(64), key=lambda j: lens[j][0])
    p, t = lens[i]
    rows = reqs[i]["idx"]
    ref_o, _ = H.oracle_row_block(reqs[i]["q"].cpu(), kp[rows].cpu(), vp[rows].cpu(), p, 1 / 16, 5, 0, max(0, t - 32), t)
    rel = H.row_rel(got[i][max(0, t - 32):t, 5].float().cpu().numpy(), ref_o)
    assert np.median(rel) < 2e-3 and (rel < 9e-3).mean() > 0.95


@pytest.mark.parametrize("hq, parts", [(24, 4), (32, 2), (16, 4)])
def test_kv_head_group_shards_concatenate_to_the_unsharded_result(pkg, cuda, hq, parts):
    """Partition by KV-head group (no exchange): every shard runs the operator on its own heads only --
    on the full pools or on a tensor-parallel slice of them -- and the shards' rows are bit-identical
    to those heads of the unsharded call, output and LSE alike."""
    from attn_kernel_lab_b200 import dist as D

    T, N, prefix, KVH = 200, 1500, 1300, 4
    q = cases.outlier_normal((T, hq, 256), 4601).to(torch.bfloat16).to(cuda)
    kp = cases.outlier_normal((N + 50, KVH, 256), 4602).to(torch.bfloat16).to(cuda)
    vp = cases.outlier_normal((N + 50, KVH, 256), 4603).to(torch.bfloat16).to(cuda)
    idx = torch.randperm(N + 50, generator=torch.Generator().manual_seed(4604))[:N].to(cuda)
    whole, whole_lse = H.fp8_extend(pkg, q, kp, vp, idx, prefix, sm_scale=1 / 16, return_lse=True)
    out = torch.full_like(q, float("nan"))
    lse = torch.full((T, hq), float("nan"), dtype=torch.float32, device=cuda)
    covered = []
    for part in range(parts):
        sharded = part % 2 == 1                       # alternate: full pools / this rank's slice of the pools
        (_, _), (klo, khi) = D.kv_head_slice(hq, KVH, part, parts)
        kps, vps = (kp[:, klo:khi].contiguous(), vp[:, klo:khi].contiguous()) if sharded else (kp, vp)
        o_s, l_s, (qlo, qhi) = D.prefill_extend_kv_head_shard(
            q, kps, vps, idx, prefix, part=part, parts=parts, out=out, lse_out=lse, pool_is_sharded=sharded,
            sm_scale=1 / 16, qk_i8=False)
        covered.append((qlo, qhi))
        assert o_s.shape == (T, hq // parts, 256)
    assert covered == [(i * hq // parts, (i + 1) * hq // parts) for i in range(parts)]
    assert torch.equal(bits(out), bits(whole)) and torch.equal(bits(lse), bits(whole_lse))
    with pytest.raises(pkg.CapabilityError):          # a shard shape is not on the production surface
        pkg.prefill_extend(q[:, :6].contiguous(), kp[:, :1].contiguous(), vp[:, :1].contiguous(), idx, prefix)
