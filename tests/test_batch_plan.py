"""The batched entry's host side, no GPU: layout arithmetic, the request table `akl_batch_plan`
writes (header, running totals, work list order), and every refusal -- all before any launch."""
import ctypes

import numpy as np
import pytest
import torch


@pytest.fixture(scope="module")
def K(pkg):
    from attn_kernel_lab_b200 import kernel

    return kernel


def _caps(K, R=4, pairs=64, qtiles=16, hq=24, hkv=4):
    return K.BatchCaps(R, pairs, qtiles, hq, hkv, 0)


def _layout(K, caps):
    lay = K.BatchLayout()
    assert K.load().akl_batch_layout(ctypes.byref(caps), ctypes.byref(lay)) == K.AKL_OK
    return lay


def _batch(K, caps, **over):
    lay = _layout(K, caps)
    b = K.Batch()
    b.caps = caps
    b.workspace, b.workspace_bytes = 1 << 30, lay.workspace_bytes
    b.table, b.table_bytes = 1 << 20, lay.table_bytes
    b.kv_dtype, b.idx_dtype = K.AKL_KV_BF16, K.AKL_IDX_I64
    b.flags, b.sm_scale = K.AKL_FLAG_ROTATE | K.AKL_FLAG_CENTER_K, 0.0625
    for k, v in over.items():
        setattr(b, k, v)
    return b, lay


def _reqs(K, shapes, **over):
    arr = (K.BatchRequest * len(shapes))()
    for i, (T, N, prefix) in enumerate(shapes):
        a = arr[i]
        a.q, a.k_pool, a.v_pool, a.idx, a.out = 0x10000, 0x20000, 0x30000, 0x40000, 0x50000
        a.lse_out = None
        a.T, a.N, a.prefix = T, N, prefix
    for k, v in over.items():
        setattr(arr[0], k, v)
    return arr


def test_struct_sizes_match_the_header(K):
    assert ctypes.sizeof(K.BatchCaps) == 24
    assert ctypes.sizeof(K.BatchLayout) == 3 * 8 + 6 * 4
    assert ctypes.sizeof(K.BatchRequest) == 6 * 8 + 4 * 4
    assert ctypes.sizeof(K.Batch) == 24 + 8 + 8 + 8 + 8 + 16


def test_layout_arithmetic_and_refusals(K):
    lib = K.load()
    lay = _layout(K, _caps(K))
    assert lay.workspace_bytes % 1024 == 0 and lay.table_bytes % 16 == 0
    # q8 + k8 + v8t tile images dominate: (24*16 + 2*4*64) * 32 KiB
    assert lay.workspace_bytes > (24 * 16 + 2 * 4 * 64) * 32768
    assert lay.table_off_geoms == 64 and lay.table_geom_stride % 8 == 0
    assert lay.table_off_items + 16 * 24 * 8 <= lay.table_bytes
    assert lay.ws_off_status + 256 <= lay.workspace_bytes
    out = K.BatchLayout()
    for bad, code in ((_caps(K, R=0), K.AKL_ERR_INVALID), (_caps(K, pairs=0), K.AKL_ERR_INVALID),
                      (_caps(K, hkv=5), K.AKL_ERR_UNSUPPORTED), (_caps(K, pairs=1 << 29), K.AKL_ERR_UNSUPPORTED)):
        assert lib.akl_batch_layout(ctypes.byref(bad), ctypes.byref(out)) == code
    assert lib.akl_batch_layout(None, ctypes.byref(out)) == K.AKL_ERR_INVALID


def test_plan_writes_header_totals_and_a_longest_first_work_list(K):
    lib = K.load()
    caps = _caps(K)
    b, lay = _batch(K, caps)
    shapes = [(130, 700, 570), (5, 5, 0), (256, 2000, 1000)]       # (T, N, prefix)
    table = np.zeros(lay.table_bytes, dtype=np.uint8)
    assert lib.akl_batch_plan(ctypes.byref(b), _reqs(K, shapes), 3, table.ctypes.data) == K.AKL_OK
    hdr = table[:64].view(np.int32)
    nt = [(n + 63) // 64 for _, n, _ in shapes]
    mt = [(t + 127) // 128 for t, _, _ in shapes]
    # attention items: 128 packed (token, head) rows of one kv head's group of 6 q heads
    pt = [(t * 6 + 127) // 128 for t, _, _ in shapes]               # 7, 1, 12
    assert hdr[1] == 3 and hdr[2] == sum(nt) * 4 and hdr[3] == sum(pt) * 4 and hdr[4] == sum(pt) * 4
    stat = table[lay.table_off_stat_totals:lay.table_off_stat_totals + 5 * 4].view(np.int32)
    assert stat.tolist() == [0, nt[0] * 4, (nt[0] + nt[1]) * 4, sum(nt) * 4, sum(nt) * 4]
    qcta = table[lay.table_off_qcta_totals:lay.table_off_qcta_totals + 5 * 4].view(np.int32)
    assert qcta.tolist() == [0, pt[0] * 4, (pt[0] + pt[1]) * 4, sum(pt) * 4, sum(pt) * 4]
    items = table[lay.table_off_items:lay.table_off_items + hdr[4] * 8].view(np.int32).reshape(-1, 2)
    # requests in order of attended pairs (2, 0, 1); inside a request deepest packed tile first, kv heads together
    assert items[:, 0].tolist() == [2] * 48 + [0] * 28 + [1] * 4
    assert (items[:4, 1] & 0xFFFF).tolist() == [11] * 4 and (items[44:48, 1] & 0xFFFF).tolist() == [0] * 4
    assert (items[:8, 1] >> 16).tolist() == [0, 1, 2, 3, 0, 1, 2, 3]
    # every (request, kv head, packed tile) exactly once
    assert len({(int(r), int(w)) for r, w in items}) == len(items)
    # planning again into the same buffer for fewer requests shrinks the counts (graph replay case)
    assert lib.akl_batch_plan(ctypes.byref(b), _reqs(K, shapes[:1]), 1, table.ctypes.data) == K.AKL_OK
    assert table[:64].view(np.int32)[1] == 1 and table[:64].view(np.int32)[4] == 7 * 4


@pytest.mark.parametrize("hq, hkv", [(16, 4), (32, 4), (8, 2), (4, 4)])
def test_work_list_counts_packed_tiles_for_every_group_size(K, hq, hkv):
    """An attention item is 128 packed (token, head) rows of one kv head's group of q heads, so a
    request of T tokens has hkv * ceil(T * group / 128) of them, each exactly once, and the Q
    quantisation totals count the same tiles."""
    lib = K.load()
    b, lay = _batch(K, _caps(K, hq=hq, hkv=hkv))
    group = hq // hkv
    shapes = [(1, 9, 8), (127, 127, 0), (129, 1000, 871), (300, 300, 0)]
    table = np.zeros(lay.table_bytes, dtype=np.uint8)
    assert lib.akl_batch_plan(ctypes.byref(b), _reqs(K, shapes), 4, table.ctypes.data) == K.AKL_OK
    hdr = table[:64].view(np.int32)
    pt = [(t * group + 127) // 128 for t, _, _ in shapes]
    assert hdr[3] == sum(pt) * hkv and hdr[4] == sum(pt) * hkv
    items = table[lay.table_off_items:lay.table_off_items + hdr[4] * 8].view(np.int32).reshape(-1, 2)
    seen = {(int(r), int(w) >> 16, int(w) & 0xFFFF) for r, w in items}
    assert seen == {(r, kvh, t) for r in range(4) for kvh in range(hkv) for t in range(pt[r])}
    # never more tiles than one 128-row tile per q head would take
    assert all(p <= group * ((t + 127) // 128) for p, (t, _, _) in zip(pt, shapes))


@pytest.mark.parametrize("shapes, over, batch_over, code", [
    ([(64, 320, 257)], {}, {}, "AKL_ERR_INVALID"),                  # prefix > N - T
    ([(0, 320, 0)], {}, {}, "AKL_ERR_INVALID"),
    ([(64, 320, 256)], dict(out=None), {}, "AKL_ERR_INVALID"),
    ([(64, 320, 256)], dict(q=0x10008), {}, "AKL_ERR_ALIGN"),
    ([(64, 320, 256)], {}, dict(sm_scale=0.0), "AKL_ERR_INVALID"),
    ([(64, 320, 256)], {}, dict(flags=16), "AKL_ERR_INVALID"),
    ([(64, 320, 256)], {}, dict(kv_dtype=9), "AKL_ERR_INVALID"),
    ([(64, 320, 256)], {}, dict(workspace=None), "AKL_ERR_INVALID"),
    ([(64, 320, 256)], {}, dict(workspace=(1 << 30) + 512), "AKL_ERR_ALIGN"),
    ([(64, 320, 256)], {}, dict(workspace_bytes=4096), "AKL_ERR_CAPACITY"),
    ([(64, 320, 256)], {}, dict(table_bytes=64), "AKL_ERR_CAPACITY"),
    ([(64, 128 * 65, 0)], {}, {}, "AKL_ERR_CAPACITY"),             # 65 pairs > 64
    ([(128 * 17, 128 * 17, 0)], {}, {}, "AKL_ERR_CAPACITY"),       # 17 q tiles > 16
    ([(1, 1, 0)] * 5, {}, {}, "AKL_ERR_CAPACITY"),                 # 5 requests > 4
    ([(64, 128 * 40, 0), (64, 128 * 25, 0)], {}, {}, "AKL_ERR_CAPACITY"),   # totals, not maxima
])
def test_plan_refuses_bad_batches_on_the_host(K, shapes, over, batch_over, code):
    lib = K.load()
    b, lay = _batch(K, _caps(K), **batch_over)
    table = np.zeros(max(int(lay.table_bytes), 64), dtype=np.uint8)
    got = lib.akl_batch_plan(ctypes.byref(b), _reqs(K, shapes, **over), len(shapes), table.ctypes.data)
    assert got == getattr(K, code)
    if batch_over:     # the launch entry checks the same batch fields before touching CUDA
        b.table = 1 << 20
        assert lib.akl_prefill_extend_batch(ctypes.byref(b), None) == getattr(K, code)
    assert lib.akl_batch_plan(ctypes.byref(b), None, 1, table.ctypes.data) in (K.AKL_ERR_INVALID, getattr(K, code))
    assert lib.akl_prefill_extend_batch(None, None) == K.AKL_ERR_INVALID


def test_python_batch_workspace_capacity_and_validation(pkg):
    cpu = torch.device("cpu")
    ws = pkg.plan_batch_workspace(cpu, max_requests=2, max_total_kv_len=1000, max_total_q_len=300,
                                  q_heads=16, kv_heads=4)
    assert (ws.q_heads, ws.kv_heads) == (16, 4)
    q = torch.zeros((100, 16, 256), dtype=torch.bfloat16)
    pool = torch.zeros((2048, 4, 256), dtype=torch.bfloat16)

    def req(n, t=100):
        return {"q": q[:t], "k_pool": pool, "v_pool": pool.clone(), "idx": torch.arange(n), "prefix": n - t,
                "out": torch.empty_like(q[:t])}

    plan = ws.plan([req(500), req(400)], sm_scale=0.0625)
    assert plan.n_requests == 2 and int(plan.table_host[:64].view(torch.int32)[1]) == 2
    ws.replan(plan, [req(300)])
    assert int(plan.table_host[:64].view(torch.int32)[1]) == 1
    with pytest.raises(pkg.WorkspaceCapacityError, match=r"outside the batch capacities"):
        ws.plan([req(900), req(900)], sm_scale=0.0625)
    with pytest.raises(pkg.WorkspaceCapacityError):
        ws.plan([req(10, 10)] * 3, sm_scale=0.0625)
    # rejection happens before anything native runs, request by request, with the field named
    with pytest.raises(pkg.CapabilityError) as info:
        pkg.prefill_extend_batch([req(500), dict(req(400), prefix=350)], workspace=ws)
    assert info.value.field == "prefix"
    with pytest.raises(RuntimeError, match=r"no CPU path"):
        pkg.prefill_extend_batch([req(500)], workspace=ws)
    with pytest.raises(ValueError, match=r"must be an int >= 1"):
        pkg.plan_batch_workspace(cpu, max_requests=0, max_total_kv_len=10, max_total_q_len=10)
    with pytest.raises(pkg.CapabilityError):
        pkg.plan_batch_workspace(cpu, max_requests=1, max_total_kv_len=10, max_total_q_len=10, q_heads=20)
