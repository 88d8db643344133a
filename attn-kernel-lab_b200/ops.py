"""Public operator entry point: validate against the declared surface, then run on the GPU.

Drop-in for the reference's src/attn_kernel_lab/ops.py: `prefill_extend`, `check_request`,
`plan_workspace` and `PrefillRequest` keep their names, arguments, validation order
(ops.py:161-407) and error classes.  What differs underneath: after validation there is ONE
native call (`akl_prefill_extend`, include/akl.h) that gathers, quantises, attends and writes
`out` / `lse_out` in their final [q_len, q_heads, ...] layout -- no scratch output and no
permute-copy (ops.py:597-609 of the reference).

Differences a caller can see, all deliberate:
  * none in the QK operand type: `qk_i8` defaults to True as in the reference (ops.py:496), an
    exact s32 QK^T on `tcgen05 kind::i8`; `qk_i8=False` is the FP8 E4M3 QK mode this build is
    measured in (`kind::f8f6f4`).
  * `idx` may be int32 as well as int64 (the reference requires int64, ops.py:248-253).
  * `prefill_extend_batch` runs a list of requests back to back on one workspace.

Nothing here initialises CUDA or loads the native library before validation has passed, so the
whole rejection surface runs on a machine with no GPU (ops.py:24-27).
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

from .capability import V1_CAPABILITY, CapabilityError, OperatorCapability, check_supported

_LSE_AVAILABLE = True
_PAGE_SIZE = 1
_MODE = "extend"
_MASK = "bottom_right_causal"

__all__ = ["PrefillRequest", "check_request", "plan_workspace", "plan_batch_workspace",
           "prefill_extend", "prefill_extend_batch"]


@dataclass(frozen=True)
class PrefillRequest:
    """Geometry implied by a validated request (ops.py:75-93)."""

    q_len: int
    q_heads: int
    kv_heads: int
    head_dim: int
    kv_len: int
    prefix: int
    sm_scale: float
    kv_dtype: str
    return_lse: bool


def _dtype_name(dtype) -> str:
    return str(dtype).rsplit(".", 1)[-1]


def _reject(message: str, *, field: str, value: object, supported: object):
    raise CapabilityError(message, field=field, value=value, supported=supported)


def _same_device(a, b) -> bool:
    if a.type != b.type:
        return False
    if a.index is None or b.index is None:
        return True
    return a.index == b.index


def _shares_storage(a, b) -> bool:
    if a.device.type == "meta" or b.device.type == "meta":
        return False
    try:
        pa = a.untyped_storage().data_ptr()
        pb = b.untyped_storage().data_ptr()
    except Exception:  # noqa: BLE001 - a tensor without storage cannot alias
        return False
    return bool(pa) and pa == pb


def check_request(q, k_pool, v_pool, idx, prefix, *, workspace=None, out=None, lse_out=None,
                  sm_scale=None, return_lse: bool = False,
                  capability: OperatorCapability = V1_CAPABILITY) -> PrefillRequest:
    """Validate one request; return its geometry.  Raises `CapabilityError` naming the field.

    Order, as in the reference (ops.py:161-407): what is needed to derive the geometry; the
    declared surface; dtypes, contiguity, lengths, devices, prefix range, sm_scale; `out`;
    `lse_out`; workspace.  Touches no device memory and loads nothing."""
    import torch

    for name, tensor in (("q", q), ("k_pool", k_pool), ("v_pool", v_pool), ("idx", idx)):
        if not isinstance(tensor, torch.Tensor):
            _reject(f"{name} must be a torch.Tensor, got {type(tensor).__name__}",
                    field=name, value=type(tensor).__name__, supported="torch.Tensor")
    if q.dim() != 3:
        _reject(f"q must be 3-D [q_len, q_heads, head_dim], got {q.dim()}-D with shape "
                f"{tuple(q.shape)}", field="q", value=tuple(q.shape),
                supported="[q_len, q_heads, head_dim]")
    if k_pool.dim() != 3:
        _reject(f"k_pool must be 3-D [pool, kv_heads, head_dim], got {k_pool.dim()}-D with shape "
                f"{tuple(k_pool.shape)}", field="k_pool", value=tuple(k_pool.shape),
                supported="[pool, kv_heads, head_dim]")
    if tuple(v_pool.shape) != tuple(k_pool.shape):
        _reject(f"v_pool shape {tuple(v_pool.shape)} must equal k_pool shape "
                f"{tuple(k_pool.shape)}: one pool geometry, two planes",
                field="v_pool", value=tuple(v_pool.shape), supported=tuple(k_pool.shape))
    q_len, q_heads, head_dim = (int(s) for s in q.shape)
    kv_heads = int(k_pool.shape[1])
    if int(k_pool.shape[2]) != head_dim:
        _reject(f"k_pool head_dim {int(k_pool.shape[2])} must equal q head_dim {head_dim}",
                field="k_pool", value=int(k_pool.shape[2]), supported=head_dim)

    if return_lse and not _LSE_AVAILABLE:
        _reject("return_lse=True is unavailable in this build", field="return_lse", value=True,
                supported=(False,))
    check_supported(head_dim=head_dim, q_heads=q_heads, kv_heads=kv_heads, page_size=_PAGE_SIZE,
                    mode=_MODE, mask=_MASK, kv_dtype=_dtype_name(k_pool.dtype),
                    return_lse=return_lse, capability=capability)

    if q.dtype != torch.bfloat16:
        _reject(f"q dtype must be bfloat16 (contract section 2), got {_dtype_name(q.dtype)}",
                field="q", value=_dtype_name(q.dtype), supported=("bfloat16",))
    if not q.is_contiguous():
        _reject("q must be contiguous: the kernels read [q_len, q_heads, head_dim] rows directly",
                field="q", value=tuple(q.stride()), supported="contiguous")
    if q_len < 1:
        _reject(f"q_len must be >= 1, got {q_len}: an empty extend must be skipped by the caller",
                field="q_len", value=q_len, supported=">= 1")
    if v_pool.dtype != k_pool.dtype:
        _reject(f"v_pool dtype {_dtype_name(v_pool.dtype)} must equal k_pool dtype "
                f"{_dtype_name(k_pool.dtype)}", field="v_pool", value=_dtype_name(v_pool.dtype),
                supported=_dtype_name(k_pool.dtype))
    if not (k_pool.is_contiguous() and v_pool.is_contiguous()):
        _reject("k_pool and v_pool must be contiguous [pool, kv_heads, head_dim]",
                field="k_pool", value=tuple(k_pool.stride()), supported="contiguous")
    if idx.dim() != 1:
        _reject(f"idx must be 1-D [kv_len] in position order, got {idx.dim()}-D with shape "
                f"{tuple(idx.shape)}", field="idx", value=tuple(idx.shape), supported="[kv_len]")
    if idx.dtype not in (torch.int64, torch.int32):
        _reject(f"idx dtype must be int64 (or int32), got {_dtype_name(idx.dtype)}",
                field="idx", value=_dtype_name(idx.dtype), supported=("int64", "int32"))
    if not idx.is_contiguous():
        _reject("idx must be contiguous", field="idx", value=tuple(idx.stride()),
                supported="contiguous")
    kv_len = int(idx.numel())
    if kv_len < 1:
        _reject("idx must name at least one kv position, got an empty index",
                field="idx", value=kv_len, supported=">= 1")
    for name, tensor in (("k_pool", k_pool), ("v_pool", v_pool), ("idx", idx)):
        if not _same_device(tensor.device, q.device):
            _reject(f"{name} is on {tensor.device} but q is on {q.device}: every operand of one "
                    "call must live on one device", field=name, value=str(tensor.device),
                    supported=str(q.device))
    if isinstance(prefix, bool) or not isinstance(prefix, int):
        _reject(f"prefix must be a Python int, got {type(prefix).__name__}: a tensor prefix would "
                "have to be read from the device to be checked",
                field="prefix", value=type(prefix).__name__, supported="int")
    if not 0 <= prefix <= kv_len - q_len:
        _reject(f"prefix={prefix} is outside [0, kv_len - q_len] = [0, {kv_len - q_len}] for "
                f"kv_len={kv_len}, q_len={q_len}: the bottom-right causal diagonal sits at offset "
                "kv_len - q_len", field="prefix", value=prefix, supported=(0, kv_len - q_len))
    if sm_scale is not None:
        if isinstance(sm_scale, bool) or not isinstance(sm_scale, (int, float)):
            _reject(f"sm_scale must be a real number or None, got {type(sm_scale).__name__}",
                    field="sm_scale", value=type(sm_scale).__name__, supported="float | None")
        if not math.isfinite(sm_scale) or sm_scale <= 0.0:
            _reject(f"sm_scale must be positive and finite, got {sm_scale!r}: it is folded into "
                    "the Q scales", field="sm_scale", value=sm_scale, supported="> 0, finite")
    if out is not None:
        if not isinstance(out, torch.Tensor):
            _reject(f"out must be a torch.Tensor or None, got {type(out).__name__}",
                    field="out", value=type(out).__name__, supported="torch.Tensor | None")
        if tuple(out.shape) != (q_len, q_heads, head_dim):
            _reject(f"out shape {tuple(out.shape)} must equal q shape "
                    f"{(q_len, q_heads, head_dim)}", field="out", value=tuple(out.shape),
                    supported=(q_len, q_heads, head_dim))
        if out.dtype != torch.bfloat16:
            _reject(f"out dtype must be bfloat16, got {_dtype_name(out.dtype)}",
                    field="out", value=_dtype_name(out.dtype), supported=("bfloat16",))
        if not out.is_contiguous():
            _reject("out must be contiguous", field="out", value=tuple(out.stride()),
                    supported="contiguous")
        if not _same_device(out.device, q.device):
            _reject(f"out is on {out.device} but q is on {q.device}", field="out",
                    value=str(out.device), supported=str(q.device))
        if _shares_storage(out, q):
            _reject("out must not overlap q storage", field="out", value="aliases q",
                    supported="a distinct allocation")
    if lse_out is not None:
        if not return_lse:
            _reject("lse_out was supplied but return_lse=False: a destination for an output that "
                    "will not be produced is a caller mistake", field="lse_out", value="supplied",
                    supported="return_lse=True")
        if not isinstance(lse_out, torch.Tensor):
            _reject(f"lse_out must be a torch.Tensor or None, got {type(lse_out).__name__}",
                    field="lse_out", value=type(lse_out).__name__, supported="torch.Tensor | None")
        if tuple(lse_out.shape) != (q_len, q_heads):
            _reject(f"lse_out shape {tuple(lse_out.shape)} must be {(q_len, q_heads)} -- one "
                    "base-2 log-sum-exp per (row, head)", field="lse_out",
                    value=tuple(lse_out.shape), supported=(q_len, q_heads))
        if lse_out.dtype != torch.float32:
            _reject(f"lse_out dtype must be float32, got {_dtype_name(lse_out.dtype)}",
                    field="lse_out", value=_dtype_name(lse_out.dtype), supported=("float32",))
        if not lse_out.is_contiguous():
            _reject("lse_out must be contiguous", field="lse_out", value=tuple(lse_out.stride()),
                    supported="contiguous")
        if not _same_device(lse_out.device, q.device):
            _reject(f"lse_out is on {lse_out.device} but q is on {q.device}", field="lse_out",
                    value=str(lse_out.device), supported=str(q.device))
    if workspace is not None:
        from .quant import FP8PrefillWorkspace

        if not isinstance(workspace, FP8PrefillWorkspace):
            got = f"{type(workspace).__module__}.{type(workspace).__qualname__}"
            _reject(f"workspace must be {FP8PrefillWorkspace.__module__}.FP8PrefillWorkspace or "
                    f"None, got {got}", field="workspace", value=got,
                    supported=f"{FP8PrefillWorkspace.__module__}.FP8PrefillWorkspace | None")
        ws_device = torch.device(workspace.device)
        if not _same_device(ws_device, q.device):
            _reject(f"workspace is on {ws_device} but q is on {q.device}", field="workspace",
                    value=str(ws_device), supported=str(q.device))

    return PrefillRequest(
        q_len=q_len, q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim, kv_len=kv_len,
        prefix=prefix,
        sm_scale=(1.0 / math.sqrt(head_dim)) if sm_scale is None else float(sm_scale),
        kv_dtype=_dtype_name(k_pool.dtype), return_lse=return_lse)


def plan_workspace(device, *, max_kv_len: int, max_q_len: int, q_heads: int | None = None,
                   kv_heads: int | None = None, need_vb16: bool = False,
                   return_lse: bool | None = None,
                   capability: OperatorCapability = V1_CAPABILITY):
    """A capacity-reserved workspace sized from the declared surface (ops.py:410-482).

    Head counts default to the largest the capability declares and are validated either way.
    The result never reallocates; a request outside the plan raises `WorkspaceCapacityError`."""
    from .quant import FP8PrefillWorkspace

    q_heads = max(capability.q_heads) if q_heads is None else int(q_heads)
    kv_heads = max(capability.kv_heads) if kv_heads is None else int(kv_heads)
    return_lse = capability.returns_lse if return_lse is None else bool(return_lse)
    check_supported(head_dim=max(capability.head_dim), q_heads=q_heads, kv_heads=kv_heads,
                    page_size=_PAGE_SIZE, mode=_MODE, mask=_MASK,
                    kv_dtype=capability.kv_dtypes[0], return_lse=return_lse,
                    capability=capability)
    if need_vb16:
        _reject("need_vb16=True: the BF16-PV fallback lane is not built; every head takes the "
                "FP8-PV path", field="need_vb16", value=True, supported=(False,))
    return FP8PrefillWorkspace(device, max_kv_len=max_kv_len, max_q_len=max_q_len,
                               q_heads=q_heads, kv_heads=kv_heads, need_vb16=False,
                               need_lse=return_lse)


def prefill_extend(q, k_pool, v_pool, idx, prefix, *, workspace=None, out=None, lse_out=None,
                   sm_scale=None, qk_i8: bool = True, rotate: bool = True, center_k: bool = True,
                   return_lse: bool = False, capability: OperatorCapability = V1_CAPABILITY,
                   check_status: bool = False):
    """Bottom-right-causal paged EXTEND attention over a page-size-1 BF16/FP16 KV pool.

    Arguments as in the reference (ops.py:485-553): `q` [q_len, q_heads, 256] BF16; `k_pool`,
    `v_pool` [pool, kv_heads, 256]; `idx` [kv_len] pool rows in position order; `prefix` in
    [0, kv_len - q_len]; query row r attends positions 0 .. prefix + r.  `workspace` from
    `plan_workspace` never reallocates; `out` / `lse_out` are written in place when given.
    Enqueues on the current CUDA stream and does not synchronise -- unless `check_status` (not in the
    reference; a debugging aid) is set: then the call waits for the stream, reads the workspace's
    status word and raises `NativeError(AKL_ERR_TIMEOUT)` if a bounded device-side wait ran out
    (the kernel then wrote NaN rows and +inf LSE instead of results).

    Returns `out`, or `(out, lse)` with `lse` [q_len, q_heads] FP32 base-2 when `return_lse`."""
    request = check_request(q, k_pool, v_pool, idx, prefix, workspace=workspace, out=out,
                            lse_out=lse_out, sm_scale=sm_scale, return_lse=return_lse,
                            capability=capability)
    if not isinstance(qk_i8, bool):
        raise TypeError(f"qk_i8 must be a bool, got {type(qk_i8).__name__}")

    # ---- everything below touches the device -------------------------------------------
    import torch

    from . import kernel as kernel_mod
    from . import quant as quant_mod

    if q.device.type != "cuda":
        raise RuntimeError(
            f"prefill_extend needs CUDA tensors, got q on {q.device}: this operator has no CPU path")
    lib = kernel_mod.load()
    ws = quant_mod.FP8PrefillWorkspace(q.device) if workspace is None else workspace
    ws.ensure(request.kv_len, request.q_len, request.q_heads, request.kv_heads)
    if out is None:
        out = torch.empty_like(q)
    lse = None
    if request.return_lse:
        lse = lse_out if lse_out is not None else torch.empty(
            (request.q_len, request.q_heads), dtype=torch.float32, device=q.device)
    call = quant_mod.make_call(
        ws, q=q, k_pool=k_pool, v_pool=v_pool, idx=idx, out=out, lse_out=lse,
        q_len=request.q_len, kv_len=request.kv_len, prefix=request.prefix,
        q_heads=request.q_heads, kv_heads=request.kv_heads, sm_scale=request.sm_scale,
        rotate=rotate, center_k=center_k, qk_i8=qk_i8)
    with torch.cuda.device(q.device):
        code = lib.akl_prefill_extend(ctypes.byref(call), torch.cuda.current_stream(q.device).cuda_stream)
    kernel_mod.check(code, "akl_prefill_extend")
    if check_status:
        _raise_on_status(ws, kernel_mod, "akl_prefill_extend")
    return (out, lse) if request.return_lse else out


def _raise_on_status(ws, kernel_mod, where: str) -> None:
    import torch

    torch.cuda.current_stream(ws.device).synchronize()
    code = ws.status()
    if code != 0:
        ws.reset_status()
        kernel_mod.check(code, where + " (device status word)")


def plan_batch_workspace(device, *, max_requests: int, max_total_kv_len: int, max_total_q_len: int,
                         q_heads: int | None = None, kv_heads: int | None = None,
                         capability: OperatorCapability = V1_CAPABILITY):
    """Capacity-reserved scratch for `prefill_extend_batch`'s native path, sized from totals over a
    batch (sum of kv lengths, sum of extend lengths).  Head counts are validated against the
    declared surface like `plan_workspace` does."""
    from .quant import FP8PrefillBatchWorkspace

    q_heads = max(capability.q_heads) if q_heads is None else int(q_heads)
    kv_heads = max(capability.kv_heads) if kv_heads is None else int(kv_heads)
    check_supported(head_dim=max(capability.head_dim), q_heads=q_heads, kv_heads=kv_heads,
                    page_size=_PAGE_SIZE, mode=_MODE, mask=_MASK, kv_dtype=capability.kv_dtypes[0],
                    return_lse=False, capability=capability)
    return FP8PrefillBatchWorkspace(device, max_requests=max_requests, max_total_kv_len=max_total_kv_len,
                                    max_total_q_len=max_total_q_len, q_heads=q_heads, kv_heads=kv_heads)


def _native_batch(requests, ws, *, sm_scale, qk_i8, rotate, center_k, return_lse, capability):
    """Validate every request, give the ones without `out` / `lse_out` their tensors, group by
    (kv dtype, idx dtype) -- one native batch per group, normally one -- and launch."""
    import torch

    from .quant import WorkspaceCapacityError

    if not isinstance(qk_i8, bool):
        raise TypeError(f"qk_i8 must be a bool, got {type(qk_i8).__name__}")
    checked = []
    for r in requests:
        checked.append(check_request(r["q"], r["k_pool"], r["v_pool"], r["idx"], r["prefix"], workspace=None,
                                     out=r.get("out"), lse_out=r.get("lse_out"), sm_scale=sm_scale,
                                     return_lse=return_lse, capability=capability))
    if not requests:
        return []
    device = requests[0]["q"].device
    if device.type != "cuda":
        raise RuntimeError(
            f"prefill_extend_batch needs CUDA tensors, got q on {device}: this operator has no CPU path")
    ws_device = torch.device(ws.device)
    for r, c in zip(requests, checked):
        if not _same_device(r["q"].device, ws_device):
            _reject(f"workspace is on {ws_device} but q is on {r['q'].device}", field="workspace",
                    value=str(ws_device), supported=str(r["q"].device))
        if (c.q_heads, c.kv_heads) != (ws.q_heads, ws.kv_heads):
            raise WorkspaceCapacityError(
                f"request heads {c.q_heads}:{c.kv_heads} differ from the batch workspace's "
                f"{ws.q_heads}:{ws.kv_heads}; the allocation never changes shape")
    filled, groups = [], {}
    for i, (r, c) in enumerate(zip(requests, checked)):
        d = dict(r)
        if d.get("out") is None:
            d["out"] = torch.empty_like(r["q"])
        if c.return_lse and d.get("lse_out") is None:
            d["lse_out"] = torch.empty((c.q_len, c.q_heads), dtype=torch.float32, device=device)
        filled.append(d)
        groups.setdefault((r["k_pool"].dtype, r["idx"].dtype), []).append(i)
    for members in groups.values():
        plan = ws.plan([filled[i] for i in members], sm_scale=checked[members[0]].sm_scale,
                       rotate=rotate, center_k=center_k, qk_i8=qk_i8)
        ws.launch(plan)
    return [(d["out"], d["lse_out"]) if c.return_lse else d["out"] for d, c in zip(filled, checked)]


_side_streams: dict = {}


def _streams_for(device, count: int):
    """`count` side streams per device, created once (stream creation is not capturable)."""
    import torch

    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    have = _side_streams.setdefault(key, [])
    while len(have) < count:
        have.append(torch.cuda.Stream(device=device))
    return have[:count]


def prefill_extend_batch(requests, *, workspace, sm_scale=None, qk_i8: bool = True, rotate: bool = True,
                         center_k: bool = True, return_lse: bool = False,
                         capability: OperatorCapability = V1_CAPABILITY):
    """Run a list of independent requests; results are exactly those of `prefill_extend` per
    request (the reference loops per request the same way,
    engines/sglang/integration/fp8_prefill/backend.py:267-289).

    `requests`: iterable of dicts with keys q, k_pool, v_pool, idx, prefix and optionally out,
    lse_out.  Every request is validated before the first launch.

    `workspace`: an `FP8PrefillBatchWorkspace` (from `plan_batch_workspace`) -> the native batched
    entry: four launches for the whole batch, per-request lengths and pointers in a device table,
    one persistent attention launch that draws (request, head, query tile) items longest first.
    One `FP8PrefillWorkspace` -> the requests run back to back on the current stream.
    A list/tuple of K workspaces -> K side streams, one workspace each; the requests are dealt to
    them longest first onto the least loaded stream (cost = attended pairs), so that the streams
    finish together.  Requests are independent units, so the gather/quantise kernels of one
    request fill the SMs that the last wave of another request's attention kernel leaves idle.  The side streams fork
    from the current stream and join it again before this function returns (event fork/join, so the
    whole batch can be captured in one CUDA graph); callers see ordinary stream semantics.
    Returns the list of results in request order."""
    requests = list(requests)
    from .quant import FP8PrefillBatchWorkspace

    if isinstance(workspace, FP8PrefillBatchWorkspace):
        return _native_batch(requests, workspace, sm_scale=sm_scale, qk_i8=qk_i8, rotate=rotate,
                             center_k=center_k, return_lse=return_lse, capability=capability)
    pool = list(workspace) if isinstance(workspace, (list, tuple)) else [workspace]
    # longest-processing-time-first assignment of requests to workspaces / streams
    cost = [int(r["q"].shape[0]) * (int(r["prefix"]) + (int(r["q"].shape[0]) + 1) / 2.0)
            if hasattr(r.get("q"), "shape") and isinstance(r.get("prefix"), int) else 0.0 for r in requests]
    load = [0.0] * len(pool)
    lane_of = [0] * len(requests)
    order = sorted(range(len(requests)), key=lambda i: (-cost[i], i))
    for i in order:
        k = min(range(len(pool)), key=lambda j: (load[j], j))
        lane_of[i] = k
        load[k] += cost[i]
    checked = []
    for i, r in enumerate(requests):       # each request against the workspace it will run on
        checked.append(check_request(r["q"], r["k_pool"], r["v_pool"], r["idx"], r["prefix"],
                                     workspace=pool[lane_of[i]], out=r.get("out"), lse_out=r.get("lse_out"),
                                     sm_scale=sm_scale, return_lse=return_lse, capability=capability))
    if len(pool) > 1 and requests:
        # outputs the caller did not supply are allocated here, on the current stream, before the
        # fork: a tensor allocated on a side stream could be handed back to that stream's
        # allocator pool while the current stream still reads it
        import torch

        requests = [dict(r) for r in requests]
        for r, c in zip(requests, checked):
            if r.get("out") is None:
                r["out"] = torch.empty_like(r["q"])
            if c.return_lse and r.get("lse_out") is None:
                r["lse_out"] = torch.empty((c.q_len, c.q_heads), dtype=torch.float32, device=r["q"].device)

    def run(r, ws):
        return prefill_extend(r["q"], r["k_pool"], r["v_pool"], r["idx"], r["prefix"], workspace=ws,
                              out=r.get("out"), lse_out=r.get("lse_out"), sm_scale=sm_scale,
                              qk_i8=qk_i8, rotate=rotate, center_k=center_k, return_lse=return_lse,
                              capability=capability)

    if len(pool) == 1 or not requests:
        return [run(r, pool[0]) for r in requests]

    import torch

    device = requests[0]["q"].device
    main = torch.cuda.current_stream(device)
    sides = _streams_for(device, len(pool))
    fork = torch.cuda.Event()
    fork.record(main)
    for side in sides:
        side.wait_event(fork)
    results = [None] * len(requests)
    for i in order:                      # each stream sees its requests longest first
        with torch.cuda.stream(sides[lane_of[i]]):
            results[i] = run(requests[i], pool[lane_of[i]])
    for side in sides:
        join = torch.cuda.Event()
        join.record(side)
        main.wait_event(join)
    return results
