"""Multi-GPU forms of the operator: one process per GPU, `torch.distributed` for the plumbing.

The reference has no multi-GPU code at all; what shards is dictated by its operator contract:

  * requests are independent units (docs/OPERATOR_CONTRACT.md:29)          -> `partition_requests`
  * q heads [j*g, (j+1)*g) read only kv head j, and every statistic is per
    kv head (docs/OPERATOR_CONTRACT.md:41-42, quant.py:516-520)            -> `kv_head_slice`
  * the KV axis of ONE long request splits if the statistics are made
    global first and the per-split (O, lse2) states are merged afterwards
    (docs/OPERATOR_CONTRACT.md:224-231, :238-242)                          -> `prefill_extend_kv_split`

Only the third form communicates.  Its collectives:
  1. SUM all-reduce of the per-tile channel-sum arrays.  Every tile is written by exactly one
     rank and is zero elsewhere, so the "sum" moves each value unchanged and the result is
     bit-identical on every rank whatever order the transport reduces in; each rank then
     performs the same ordered additions (tiles inside a 32768-row slab, then slabs) as a
     single GPU would.  A SUM all-reduce of overlapping partial sums is NOT used: its order
     is unspecified.
  2. MAX all-reduce of the raw per-head V amax (order-independent).
  3. an all-to-all of (O_i, lse_i) row slices -- a reduce-scatter over query rows whose
     reduction is the `akl_merge_states` kernel, run on data that has landed in local HBM.

No kernel of this library waits on another rank; ranks only meet inside the collectives.
"""
from __future__ import annotations

import ctypes

import torch

from . import kernel as _kernel
from . import quant as _quant

SPLIT_GRANULE = 1024   # KV-axis split points are multiples of this many positions (64-tile aligned)


# ------------------------------------------------------------------ host-side planning
def partition_requests(costs, world: int):
    """Greedy longest-processing-time assignment of request indices to `world` ranks.
    `costs` are per-request FLOPs (4*Hq*D*T*(prefix+(T+1)/2)).  Returns world lists."""
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    loads = [0.0] * world
    bins = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (loads[j], j))
        bins[r].append(i)
        loads[r] += costs[i]
    for b in bins:
        b.sort()
    return bins


def kv_head_slice(q_heads: int, kv_heads: int, part: int, parts: int):
    """Head ranges of one of `parts` KV-head groups: ((q_lo, q_hi), (kv_lo, kv_hi))."""
    if kv_heads % parts:
        raise ValueError(f"kv_heads={kv_heads} does not split into {parts} groups")
    per = kv_heads // parts
    g = q_heads // kv_heads
    return (part * per * g, (part + 1) * per * g), (part * per, (part + 1) * per)


def prefill_extend_kv_head_shard(q, k_pool, v_pool, idx, prefix, *, part: int, parts: int, out=None, lse_out=None,
                                 workspace=None, pool_is_sharded: bool = False, **kwargs):
    """One KV-head-group shard of a request: the part of the work rank `part` of `parts` owns.

    `q` is the request's full query tensor [T, Hq, 256]; the shard attends its q heads
    `kv_head_slice(...)[0]` to its kv heads.  `k_pool` / `v_pool` are either the full pools
    [pool, Hkv, 256] (the shard's heads are taken out of them) or, with `pool_is_sharded`, this rank's
    own [pool, Hkv / parts, 256] slice, as a tensor-parallel engine keeps it.  `out` / `lse_out`, when
    given, are the FULL [T, Hq, 256] / [T, Hq] tensors and only this shard's heads are written.
    Returns (out_shard [T, Hq/parts, 256], lse_shard or None, (q_head_lo, q_head_hi)).

    No collective: query heads read one kv head, and every statistic is per kv head, so the shard's
    rows are bit-identical to the same heads of the unsharded call."""
    from . import ops
    from .capability import KV_HEAD_SHARD_CAPABILITY

    Hq = int(q.shape[1])
    Hkv_total = int(k_pool.shape[1]) * (parts if pool_is_sharded else 1)
    (qlo, qhi), (klo, khi) = kv_head_slice(Hq, Hkv_total, part, parts)
    q_s = q[:, qlo:qhi].contiguous()
    if pool_is_sharded:
        kp, vp = k_pool, v_pool
    else:
        kp, vp = k_pool[:, klo:khi].contiguous(), v_pool[:, klo:khi].contiguous()
    want_lse = bool(kwargs.pop("return_lse", lse_out is not None))
    res = ops.prefill_extend(q_s, kp, vp, idx, prefix, workspace=workspace, return_lse=want_lse,
                             capability=KV_HEAD_SHARD_CAPABILITY, **kwargs)
    o_s, l_s = res if want_lse else (res, None)
    if out is not None:
        out[:, qlo:qhi].copy_(o_s)
    if lse_out is not None:
        lse_out[:, qlo:qhi].copy_(l_s)
    return o_s, l_s, (qlo, qhi)


def kv_split_ranges(n_total: int, world: int, granule: int = SPLIT_GRANULE):
    """Cut [0, n_total) into `world` contiguous ranges whose interior boundaries are
    multiples of `granule`.  Trailing ranks may be empty when n_total is small."""
    blocks = (n_total + granule - 1) // granule
    base, extra = divmod(blocks, world)
    out, lo = [], 0
    for r in range(world):
        nb = base + (1 if r < extra else 0)
        hi = min(n_total, lo + nb * granule)
        out.append((lo, hi))
        lo = hi
    return out


def row_slices(rows: int, world: int):
    """Contiguous ownership of query rows for the merge: rank r owns rows [lo_r, hi_r)."""
    per = (rows + world - 1) // world
    return [(min(rows, r * per), min(rows, (r + 1) * per)) for r in range(world)]


# ------------------------------------------------------------------ merge (single device)
def merge_states(parts_o, parts_lse, out=None, lse_out=None):
    """Merge per-split partial states with the `akl_merge_states` kernel.

    parts_o: list of [rows, 256] (or [T, H, 256]) BF16 tensors on one device; parts_lse: list of
    matching FP32 base-2 LSE tensors.  Returns (out, lse)."""
    lib = _kernel.load()
    dev = parts_o[0].device
    rows = parts_lse[0].numel()
    if out is None:
        out = torch.empty_like(parts_o[0])
    if lse_out is None:
        lse_out = torch.empty_like(parts_lse[0])
    po = torch.tensor([p.data_ptr() for p in parts_o], dtype=torch.int64, device=dev)
    pl = torch.tensor([p.data_ptr() for p in parts_lse], dtype=torch.int64, device=dev)
    m = _kernel.Merge(po.data_ptr(), pl.data_ptr(), out.data_ptr(), lse_out.data_ptr(),
                      len(parts_o), rows)
    with torch.cuda.device(dev):
        code = lib.akl_merge_states(ctypes.byref(m), torch.cuda.current_stream(dev).cuda_stream)
    _kernel.check(code, "akl_merge_states")
    # the pointer tables must outlive the launch on this stream
    po.record_stream(torch.cuda.current_stream(dev))
    pl.record_stream(torch.cuda.current_stream(dev))
    return out, lse_out


# ------------------------------------------------------------------ KV-axis split of one request
def kv_split_local(ws, q, k_pool, v_pool, idx_local, prefix: int, *, n_total: int, kv_lo: int,
                   sm_scale: float, rotate: bool = True, center_k: bool = True, qk_i8: bool = False,
                   all_reduce_sum=None, all_reduce_max=None, phases=None):
    """One rank's share of a KV-split request: statistics made global through the two
    callbacks, then transform + attention over local positions [kv_lo, kv_lo + len(idx_local)).

    Returns (O_i [T, Hq, 256] BF16 normalised with the V mean added, lse_i [T, Hq] FP32).
    `all_reduce_sum(t)` / `all_reduce_max(t)` reduce a tensor in place across ranks (identity
    for a single-rank emulation that shares the arrays).  `phases(name, call)` runs one phase
    entry point; the default calls the native library on the current stream (host-logic tests
    on CPU ranks pass a stand-in that fills the same workspace regions)."""
    if phases is None:
        lib = _kernel.load()
        st = torch.cuda.current_stream(q.device).cuda_stream

        def phases(name, call):
            _kernel.check(getattr(lib, name)(ctypes.byref(call), st), name)
    T, Hq = int(q.shape[0]), int(q.shape[1])
    Hkv = int(k_pool.shape[1])
    n_local = int(idx_local.numel())
    ntg = (n_total + _quant.BLK - 1) // _quant.BLK
    ws.ensure(n_total, T, Hq, Hkv)
    out = torch.empty_like(q)
    lse = torch.empty((T, Hq), dtype=torch.float32, device=q.device)
    have = n_local > 0
    if not have:
        # a rank without keys still takes part in the collectives and emits weight-zero states
        idx_local = torch.zeros(1, dtype=torch.int64, device=q.device)
    call = _quant.make_call(
        ws, q=q, k_pool=k_pool, v_pool=v_pool, idx=idx_local, out=out, lse_out=lse, q_len=T,
        kv_len=max(n_local, 1), prefix=prefix, q_heads=Hq, kv_heads=Hkv, sm_scale=sm_scale,
        rotate=rotate, center_k=center_k, qk_i8=qk_i8, kv_pos0=kv_lo, n_total=n_total,
        tile0_global=kv_lo // _quant.BLK, ntiles_global=ntg)
    ktsum, vtsum = ws.view("ktsum"), ws.view("vtsum")
    ktsum[:ntg].zero_()
    vtsum[:ntg].zero_()
    if have:
        phases("akl_kv_tile_stats", call)
    if all_reduce_sum is not None:
        all_reduce_sum(ktsum[:ntg])
        all_reduce_sum(vtsum[:ntg])
    if have:
        phases("akl_kv_means", call)
    else:
        ws.view("vsmax").zero_()
    if all_reduce_max is not None:
        all_reduce_max(ws.view("vsmax"))
    if not have:
        lse.fill_(float("-inf"))
        out.zero_()
        return out, lse
    for fn in ("akl_kv_scales", "akl_kv_transform", "akl_quantize_q", "akl_attention"):
        phases(fn, call)
    return out, lse


def prefill_extend_kv_split(ws, q, k_pool, v_pool, idx_local, prefix: int, *, n_total: int,
                            kv_lo: int, sm_scale: float, group=None, rotate: bool = True,
                            center_k: bool = True, qk_i8: bool = False, phases=None, merge=None):
    """KV-axis split of one long request across the ranks of `group` (default: world).

    Every rank passes the full `q`, its own slice of the page table (`idx_local`, global
    positions [kv_lo, kv_lo + len)), and pools that hold at least those rows.  Returns this
    rank's slice of the merged result: (out [rows_r, Hq, 256] BF16, lse [rows_r, Hq] FP32,
    (row_lo, row_hi))."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)

    def ar_sum(t):
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)

    def ar_max(t):
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)

    o_i, lse_i = kv_split_local(ws, q, k_pool, v_pool, idx_local, prefix, n_total=n_total,
                                kv_lo=kv_lo, sm_scale=sm_scale, rotate=rotate, center_k=center_k,
                                qk_i8=qk_i8, all_reduce_sum=ar_sum, all_reduce_max=ar_max, phases=phases)
    return exchange_and_merge(o_i, lse_i, group=group, merge=merge)


_recv_cache: dict = {}


def _staging(o_send, l_send):
    """Receive buffers for the exchange, kept per (device, shape): a long prefill calls this once per
    layer with the same shapes, and the previous call's merge has consumed them in stream order."""
    key = (o_send.device, tuple(o_send.shape), o_send.dtype)
    bufs = _recv_cache.get(key)
    if bufs is None:
        if len(_recv_cache) > 8:
            _recv_cache.clear()
        bufs = (torch.empty_like(o_send), torch.empty_like(l_send))
        _recv_cache[key] = bufs
    return bufs


def exchange_and_merge(o_i, lse_i, *, group=None, merge=None):
    """Reduce-scatter over query rows of the per-rank partial states.

    Rank r ends up with rows `row_slices(T, world)[r]` of the merged result.  The transport is
    one all-to-all per tensor; the reduction is `merge` (default: the `akl_merge_states`
    kernel) over the partials once they are in local memory."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    merge = merge_states if merge is None else merge
    T, Hq, D = o_i.shape
    slices = row_slices(T, world)
    per = slices[0][1] - slices[0][0]
    if world * per == T and o_i.is_contiguous() and lse_i.is_contiguous():
        o_send, l_send = o_i, lse_i          # rows divide evenly: the partial states are the send buffers
    else:
        # pad rows to world * per so the all-to-all is regular
        o_send = torch.zeros((world * per, Hq, D), dtype=o_i.dtype, device=o_i.device)
        l_send = torch.full((world * per, Hq), float("-inf"), dtype=torch.float32, device=o_i.device)
        o_send[:T] = o_i
        l_send[:T] = lse_i
    o_recv, l_recv = _staging(o_send, l_send)
    dist.all_to_all_single(o_recv, o_send, group=group)
    dist.all_to_all_single(l_recv, l_send, group=group)
    parts_o = [o_recv[r * per:(r + 1) * per] for r in range(world)]
    parts_l = [l_recv[r * per:(r + 1) * per] for r in range(world)]
    out, lse = merge(parts_o, parts_l)
    lo, hi = slices[rank]
    return out[:hi - lo], lse[:hi - lo], (lo, hi)
