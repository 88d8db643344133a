"""Workspace and preprocessing entry points of the operator.

Host-side mirror of the reference's src/attn_kernel_lab/quant.py: the same public names
(`FP8PrefillWorkspace`, `CapacityPlan`, `WorkspaceCapacityError`, `gather_quantize_kv`,
`quantize_q`, `BLK`, `MPAD`, `SLAB`, `FP8_MAX`) with the same meaning, but

  * the workspace is ONE device allocation carved by the native `akl_workspace_layout`
    instead of a dictionary of tensors (quant.py:303-321), and
  * every arithmetic step runs in the CUDA kernels of csrc/akl_prep.cu instead of ~14
    tensor-library launches (quant.py:433-695).

Byte layout of the quantised tiles is this build's (layout version 2: 128-byte-swizzled
tensor-core tile images); `q8_logical` / `k8_logical` / `v8_logical` return the position-order
bytes the reference's buffers hold, which is what parity tests compare.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import kernel as _kernel

HEAD_DIM = 256
BLK = 64       # kv quantisation tile (quant.py:80)
MPAD = 128     # query padding granule (quant.py:86)
SLAB = 32768   # statistics slab, numerics-visible (quant.py:87-91)
FP8_MAX = 448.0
DECLARED_Q_HEADS = 24
DECLARED_KV_HEADS = 4


def _ceil_to(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class WorkspaceCapacityError(RuntimeError):
    """A capacity-reserved workspace was asked for more than its plan.

    Not a `CapabilityError` on purpose (quant.py:164-172): a plan miss under a captured CUDA
    graph must fail the request, not be routed around."""


@dataclass(frozen=True)
class CapacityPlan:
    """Maxima a reserved workspace was sized for, with the padded geometry (quant.py:175-196)."""

    max_kv_len: int
    max_q_len: int
    q_heads: int
    kv_heads: int
    need_vb16: bool
    need_lse: bool
    npad: int
    ntmax: int
    mpad: int

    def admits(self, kv_len: int, q_len: int) -> bool:
        return 1 <= kv_len <= self.max_kv_len and 1 <= q_len <= self.max_q_len


_REGIONS = ("q8", "qscale", "k8", "v8t", "kscale", "vst", "vlog2r", "vinvr", "vam", "vscale",
            "vsmax", "kmean", "vmean", "ktsum", "vtsum", "vtmax", "vtmin", "status")


class FP8PrefillWorkspace:
    """Device scratch for the operator: grown on demand, or reserved once and locked.

    `FP8PrefillWorkspace(device)` grows when a request needs more (eager use only).
    `FP8PrefillWorkspace(device, max_kv_len=..., max_q_len=...)` or `.reserve(...)` sizes it
    once; afterwards a request outside the plan raises `WorkspaceCapacityError` and no address
    ever moves -- the property CUDA graph capture needs (quant.py:253-336)."""

    def __init__(self, device, *, max_kv_len=None, max_q_len=None,
                 q_heads: int = DECLARED_Q_HEADS, kv_heads: int = DECLARED_KV_HEADS,
                 need_vb16: bool = False, need_lse: bool = True):
        self.device = torch.device(device)
        self._plan: CapacityPlan | None = None
        self._buf: torch.Tensor | None = None      # raw allocation
        self._base: torch.Tensor | None = None     # 1024-byte aligned view
        self._layout = None
        self._dims = None                          # (max_kv_len, max_q_len, q_heads, kv_heads)
        if max_kv_len is not None or max_q_len is not None:
            if max_kv_len is None or max_q_len is None:
                raise ValueError(
                    "capacity mode needs BOTH max_kv_len and max_q_len: pinning one dimension "
                    "and growing the other still reallocates")
            self.reserve(max_kv_len, max_q_len, q_heads=q_heads, kv_heads=kv_heads,
                         need_vb16=need_vb16, need_lse=need_lse)

    # ------------------------------------------------------------------ planning
    @property
    def capacity(self) -> CapacityPlan | None:
        return self._plan

    def reserve(self, max_kv_len: int, max_q_len: int, *, q_heads: int = DECLARED_Q_HEADS,
                kv_heads: int = DECLARED_KV_HEADS, need_vb16: bool = False,
                need_lse: bool = True) -> CapacityPlan:
        for name, value in (("max_kv_len", max_kv_len), ("max_q_len", max_q_len),
                            ("q_heads", q_heads), ("kv_heads", kv_heads)):
            if isinstance(value, bool) or not isinstance(value, int) or value < 1:
                raise ValueError(f"{name} must be an int >= 1, got {value!r}")
        if q_heads % kv_heads:
            raise ValueError(f"q_heads={q_heads} must be divisible by kv_heads={kv_heads}")
        if need_vb16:
            raise ValueError("need_vb16: the BF16-PV fallback lane is not part of this build "
                             "(the declared surface is all-FP8-PV)")
        self._plan = None
        self._allocate(max_kv_len, max_q_len, q_heads, kv_heads)
        self._plan = CapacityPlan(
            max_kv_len=max_kv_len, max_q_len=max_q_len, q_heads=q_heads, kv_heads=kv_heads,
            need_vb16=False, need_lse=need_lse, npad=_ceil_to(max_kv_len, BLK),
            ntmax=_ceil_to(max_kv_len, BLK) // BLK, mpad=_ceil_to(max_q_len, MPAD))
        return self._plan

    def release_capacity(self) -> None:
        """Back to grow-on-demand; the allocation is kept (quant.py:338-344)."""
        self._plan = None

    def _allocate(self, max_kv_len, max_q_len, q_heads, kv_heads) -> None:
        layout = _kernel.workspace_layout(max_kv_len, max_q_len, q_heads, kv_heads)
        total = int(layout.total_bytes)
        buf = torch.empty(total + 1024, dtype=torch.uint8, device=self.device)
        shift = (-buf.data_ptr()) % 1024
        self._buf = buf
        self._base = buf[shift:shift + total]
        self._layout = layout
        self._dims = (max_kv_len, max_q_len, q_heads, kv_heads)
        self.view("status").zero_()

    def ensure(self, kv_len: int, q_len: int, q_heads: int, kv_heads: int) -> None:
        """Make room for a request, or refuse if the workspace is locked to a smaller plan."""
        if self._dims is not None:
            mk, mq, hq, hkv = self._dims
            if kv_len <= mk and q_len <= mq and hq == q_heads and hkv == kv_heads:
                return
        if self._plan is not None:
            raise WorkspaceCapacityError(
                f"request (kv_len={kv_len}, q_len={q_len}, heads={q_heads}:{kv_heads}) is outside "
                f"the capacity plan {self._plan}. Growing would move the device addresses a "
                "captured CUDA graph holds. Re-reserve at larger maxima, or call "
                "release_capacity() to go back to growing on demand.")
        same_heads = self._dims is not None and self._dims[2:] == (q_heads, kv_heads)
        mk, mq = (self._dims[0], self._dims[1]) if same_heads else (0, 0)
        old = {name: self.view(name) for name in _REGIONS} if same_heads else {}
        self._allocate(max(mk, kv_len), max(mq, q_len), q_heads, kv_heads)
        # growing keeps what earlier phase calls wrote (each region grows along its capacity axes)
        for name, src in old.items():
            self.view(name)[tuple(slice(0, n) for n in src.shape)].copy_(src)

    # ------------------------------------------------------------------ access
    @property
    def layout(self):
        return self._layout

    @property
    def dims(self):
        return self._dims

    def base_ptr(self) -> int:
        return self._base.data_ptr()

    def nbytes(self) -> int:
        return self._base.numel()

    def buffer_pointers(self) -> dict[str, int]:
        """{region name: device address}; stable across calls in capacity mode (quant.py:346-353)."""
        if self._layout is None:
            return {}
        base = self.base_ptr()
        return {name: base + int(getattr(self._layout, "off_" + name)) for name in _REGIONS}

    def view(self, name: str) -> torch.Tensor:
        """Typed view of one named region at its capacity shape."""
        L = self._layout
        mk, mq, hq, hkv = self._dims
        f32 = torch.float32
        shapes = {
            "q8": ((hq, L.mtiles, 2, 128, 128), torch.uint8),
            "qscale": ((hq, L.mtiles * 128), f32),
            "k8": ((hkv, L.npairs, 2, 128, 128), torch.uint8),
            "v8t": ((hkv, L.npairs, 256, 128), torch.uint8),
            "kscale": ((hkv, L.ntiles), f32), "vst": ((hkv, L.ntiles), f32),
            "vlog2r": ((hkv, L.ntiles), f32), "vinvr": ((hkv, L.ntiles), f32),
            "vam": ((hkv, L.ntiles), f32),
            "vscale": ((hkv,), f32), "vsmax": ((hkv,), f32),
            "kmean": ((hkv, HEAD_DIM), f32), "vmean": ((hkv, HEAD_DIM), f32),
            "ktsum": ((L.ntiles, hkv, HEAD_DIM), f32), "vtsum": ((L.ntiles, hkv, HEAD_DIM), f32),
            "vtmax": ((hkv, L.ntiles, HEAD_DIM), f32), "vtmin": ((hkv, L.ntiles, HEAD_DIM), f32),
            "status": ((64,), torch.int32),
        }
        shape, dtype = shapes[name]
        off = int(getattr(L, "off_" + name))
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        return self._base[off:off + nbytes].view(dtype).view(shape)

    def status(self) -> int:
        """First device-side error code recorded since allocation or the last reset (synchronises)."""
        return int(self.view("status")[0].item())

    def reset_status(self) -> None:
        self.view("status").zero_()

    # position-order bytes, as the reference's buffers hold them ---------------------------
    def q8_logical(self, q_len: int) -> torch.Tensor:
        """[Hq, Mpad, 256] uint8 (quant.py:457)."""
        mt = _ceil_to(q_len, MPAD) // MPAD
        img = self.view("q8")[:, :mt]
        return _unswizzle_planes(img).reshape(img.shape[0], mt * 128, HEAD_DIM)

    def k8_logical(self, kv_len: int) -> torch.Tensor:
        """[Hkv, Npad, 256] uint8, Npad = ceil64(kv_len) (quant.py:509)."""
        npad = _ceil_to(kv_len, BLK)
        npairs = _ceil_to(kv_len, 128) // 128
        img = self.view("k8")[:, :npairs]
        return _unswizzle_planes(img).reshape(img.shape[0], npairs * 128, HEAD_DIM)[:, :npad]

    def v8_logical(self, kv_len: int) -> torch.Tensor:
        """[Hkv, Npad, 256] uint8 in position order (the reference's vt8 without its SIGMA
        permutation and transpose, quant.py:625-635)."""
        npad = _ceil_to(kv_len, BLK)
        npairs = _ceil_to(kv_len, 128) // 128
        img = self.view("v8t")[:, :npairs]                       # [Hkv, np, 256 d, 128 key]
        rows = torch.arange(256, device=img.device)[:, None]
        cols = torch.arange(128, device=img.device)[None, :]
        src = (((cols >> 4) ^ (rows & 7)) << 4) | (cols & 15)    # stored byte column
        dk = torch.gather(img, 3, src.expand(img.shape[0], npairs, 256, 128))
        return dk.permute(0, 1, 3, 2).reshape(img.shape[0], npairs * 128, HEAD_DIM)[:, :npad]


class BatchPlan:
    """A request table as `akl_batch_plan` wrote it, in pinned host memory, plus what is needed to
    launch it.  `FP8PrefillBatchWorkspace.launch(plan)` copies it to the device and enqueues the
    four kernels; a captured CUDA graph that holds that copy re-reads this host buffer at every
    replay, so `FP8PrefillBatchWorkspace.replan(plan, requests)` followed by a replay runs the new
    lengths and tensors without re-capturing."""

    def __init__(self, table_host, batch, n_requests):
        self.table_host = table_host
        self.batch = batch
        self.n_requests = n_requests


class FP8PrefillBatchWorkspace:
    """Capacity-reserved scratch for the batched entry `akl_prefill_extend_batch`: ONE device
    allocation shared by all requests of a batch (each request's tiles are packed behind the
    previous request's) and one device copy of the request table.  Sized once from totals; never
    reallocates.  A batch that needs more raises `WorkspaceCapacityError`.

    The capacities are totals over a batch: `max_total_kv_len` >= sum of kv lengths and
    `max_total_q_len` >= sum of extend lengths (each request rounds up to whole 128-row tiles;
    room for that rounding is added per request)."""

    def __init__(self, device, *, max_requests: int, max_total_kv_len: int, max_total_q_len: int,
                 q_heads: int = DECLARED_Q_HEADS, kv_heads: int = DECLARED_KV_HEADS):
        for name, value in (("max_requests", max_requests), ("max_total_kv_len", max_total_kv_len),
                            ("max_total_q_len", max_total_q_len), ("q_heads", q_heads), ("kv_heads", kv_heads)):
            if isinstance(value, bool) or not isinstance(value, int) or value < 1:
                raise ValueError(f"{name} must be an int >= 1, got {value!r}")
        if q_heads % kv_heads:
            raise ValueError(f"q_heads={q_heads} must be divisible by kv_heads={kv_heads}")
        self.device = torch.device(device)
        self.caps = _kernel.BatchCaps(
            max_requests, _ceil_to(max_total_kv_len, 128) // 128 + max_requests,
            _ceil_to(max_total_q_len, MPAD) // MPAD + max_requests, q_heads, kv_heads, 0)
        lay = _kernel.BatchLayout()
        _kernel.check(_kernel.load().akl_batch_layout(ctypes.byref(self.caps), ctypes.byref(lay)),
                      "akl_batch_layout")
        self._ws_bytes, self._table_bytes = int(lay.workspace_bytes), int(lay.table_bytes)
        buf = torch.empty(self._ws_bytes + 1024, dtype=torch.uint8, device=self.device)
        shift = (-buf.data_ptr()) % 1024
        self._buf = buf
        self._base = buf[shift:shift + self._ws_bytes]
        self._table_dev = torch.empty(self._table_bytes + 16, dtype=torch.uint8, device=self.device)
        tshift = (-self._table_dev.data_ptr()) % 16
        self._table = self._table_dev[tshift:tshift + self._table_bytes]
        self.layout = lay
        self._status = self._base[int(lay.ws_off_status):int(lay.ws_off_status) + 256].view(torch.int32)
        self._status.zero_()
        self._held = []          # host tables a captured graph still reads

    @property
    def q_heads(self) -> int:
        return int(self.caps.q_heads)

    @property
    def kv_heads(self) -> int:
        return int(self.caps.kv_heads)

    def nbytes(self) -> int:
        return self._ws_bytes + self._table_bytes

    def base_ptr(self) -> int:
        return self._base.data_ptr()

    def status(self) -> int:
        """First device-side error code recorded since allocation or the last reset (synchronises)."""
        return int(self._status[0].item())

    def reset_status(self) -> None:
        self._status.zero_()

    def admits(self, n_requests: int, total_kv_len: int, total_q_len: int) -> bool:
        """Whether a batch with these totals certainly fits (every request rounds up to whole
        128-row tiles, so one tile per request is held back)."""
        return (n_requests <= self.caps.max_requests
                and _ceil_to(total_kv_len, 128) // 128 + n_requests <= self.caps.max_total_kv_pairs
                and _ceil_to(total_q_len, MPAD) // MPAD + n_requests <= self.caps.max_total_q_tiles)

    # ------------------------------------------------------------------ planning
    def _batch_struct(self, kv_dtype, idx_dtype, flags, sm_scale):
        b = _kernel.Batch()
        b.caps = self.caps
        b.workspace, b.workspace_bytes = self._base.data_ptr(), self._ws_bytes
        b.table, b.table_bytes = self._table.data_ptr(), self._table_bytes
        b.kv_dtype, b.idx_dtype, b.flags, b.sm_scale = kv_dtype, idx_dtype, flags, float(sm_scale)
        return b

    @staticmethod
    def _request_array(requests):
        arr = (_kernel.BatchRequest * max(1, len(requests)))()
        for i, r in enumerate(requests):
            a = arr[i]
            a.q, a.k_pool, a.v_pool = r["q"].data_ptr(), r["k_pool"].data_ptr(), r["v_pool"].data_ptr()
            a.idx, a.out = r["idx"].data_ptr(), r["out"].data_ptr()
            lse = r.get("lse_out")
            a.lse_out = lse.data_ptr() if lse is not None else None
            a.T, a.N, a.prefix = int(r["q"].shape[0]), int(r["idx"].shape[0]), int(r["prefix"])
        return arr

    def _fill(self, table_host, batch, requests):
        arr = self._request_array(requests)
        code = _kernel.load().akl_batch_plan(ctypes.byref(batch), arr, len(requests), table_host.data_ptr())
        if code == _kernel.AKL_ERR_CAPACITY:
            raise WorkspaceCapacityError(
                f"batch of {len(requests)} requests (sum kv {sum(int(r['idx'].shape[0]) for r in requests)}, "
                f"sum q {sum(int(r['q'].shape[0]) for r in requests)}) is outside the batch capacities "
                f"(requests {self.caps.max_requests}, kv pairs {self.caps.max_total_kv_pairs}, "
                f"q tiles {self.caps.max_total_q_tiles}); the allocation never grows")
        _kernel.check(code, "akl_batch_plan")

    def plan(self, requests, *, sm_scale: float, rotate: bool = True, center_k: bool = True,
             qk_i8: bool = False) -> BatchPlan:
        """Host-side only: pack `requests` (dicts with q, k_pool, v_pool, idx, prefix, out and
        optionally lse_out; one kv dtype and one idx dtype) into a fresh pinned request table."""
        requests = list(requests)
        if not requests:
            raise ValueError("an empty batch has nothing to plan")
        flags = ((_kernel.AKL_FLAG_ROTATE if rotate else 0) | (_kernel.AKL_FLAG_CENTER_K if center_k else 0)
                 | (_kernel.AKL_FLAG_QK_I8 if qk_i8 else 0))
        batch = self._batch_struct(_dtype_code(requests[0]["k_pool"]), _idx_code(requests[0]["idx"]), flags, sm_scale)
        pin = self.device.type == "cuda"
        table_host = torch.empty(self._table_bytes, dtype=torch.uint8, pin_memory=pin)
        self._fill(table_host, batch, requests)
        return BatchPlan(table_host, batch, len(requests))

    def replan(self, plan: BatchPlan, requests) -> None:
        """Rewrite `plan`'s host table in place for other requests (same dtypes and modes)."""
        requests = list(requests)
        self._fill(plan.table_host, plan.batch, requests)
        plan.n_requests = len(requests)

    def upload(self, plan: BatchPlan) -> None:
        """Copy the table to the device (stream-ordered, from pinned memory)."""
        self._table.copy_(plan.table_host, non_blocking=True)
        if torch.cuda.is_current_stream_capturing():
            self._held.append(plan)      # the graph's copy node reads this host buffer at replay

    def launch(self, plan: BatchPlan, phases: int = _kernel.AKL_BATCH_ALL, upload: bool = True) -> None:
        """Copy the table to the device and enqueue the batch's kernels on the current stream
        (`phases`: a subset, AKL_BATCH_* bits, for per-phase timing)."""
        if upload:
            self.upload(plan)
        with torch.cuda.device(self.device):
            code = _kernel.load().akl_prefill_extend_batch_phases(ctypes.byref(plan.batch), phases,
                                                                  _stream(self.device))
        _kernel.check(code, "akl_prefill_extend_batch_phases")


def _unswizzle_planes(img: torch.Tensor) -> torch.Tensor:
    """[..., 2, 128 rows, 128 B swizzled] -> [..., 128 rows, 256 B]."""
    rows = torch.arange(128, device=img.device)[:, None]
    cols = torch.arange(128, device=img.device)[None, :]
    src = (((cols >> 4) ^ (rows & 7)) << 4) | (cols & 15)
    planes = torch.gather(img, img.dim() - 1, src.expand(img.shape))
    return torch.cat([planes[..., 0, :, :], planes[..., 1, :, :]], dim=-1)


# ---------------------------------------------------------------------- native calls
def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _kernel.AKL_KV_BF16
    if t.dtype == torch.float16:
        return _kernel.AKL_KV_FP16
    raise TypeError(f"kv pool dtype {t.dtype} is not bfloat16/float16")


def _idx_code(t: torch.Tensor) -> int:
    if t.dtype == torch.int64:
        return _kernel.AKL_IDX_I64
    if t.dtype == torch.int32:
        return _kernel.AKL_IDX_I32
    raise TypeError(f"idx dtype {t.dtype} is not int64/int32")


def make_call(ws: FP8PrefillWorkspace, *, q=None, k_pool, v_pool, idx, out=None, lse_out=None,
              q_len: int, kv_len: int, prefix: int, q_heads: int, kv_heads: int, sm_scale: float,
              rotate: bool = True, center_k: bool = True, qk_i8: bool = False, kv_pos0: int = 0,
              n_total: int = 0, tile0_global: int = 0, ntiles_global: int = 0) -> "_kernel.Call":
    """Fill an `akl_call_t` from tensors (pointers only; nothing is copied or launched)."""
    mk, mq, hq, hkv = ws.dims
    c = _kernel.Call()
    c.q = q.data_ptr() if q is not None else None
    c.k_pool = k_pool.data_ptr()
    c.v_pool = v_pool.data_ptr()
    c.idx = idx.data_ptr()
    c.out = out.data_ptr() if out is not None else None
    c.lse_out = lse_out.data_ptr() if lse_out is not None else None
    c.workspace = ws.base_ptr()
    c.workspace_bytes = ws.nbytes()
    c.plan = _kernel.Plan(mk, mq, hq, hkv)
    c.T, c.N, c.prefix = q_len, kv_len, prefix
    c.q_heads, c.kv_heads = q_heads, kv_heads
    c.kv_dtype = _dtype_code(k_pool)
    c.idx_dtype = _idx_code(idx) if idx.dtype in (torch.int64, torch.int32) else _kernel.AKL_IDX_I64
    c.flags = ((_kernel.AKL_FLAG_ROTATE if rotate else 0) | (_kernel.AKL_FLAG_CENTER_K if center_k else 0)
               | (_kernel.AKL_FLAG_QK_I8 if qk_i8 else 0))
    c.sm_scale = float(sm_scale)
    c.kv_pos0, c.n_total = kv_pos0, n_total
    c.tile0_global, c.ntiles_global = tile0_global, ntiles_global
    return c


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def gather_quantize_kv(ws: FP8PrefillWorkspace, k_buffer, v_buffer, idx, need_vt8: bool = True,
                       need_vb16: bool = False, center_k: bool = True, qk_i8: bool = True,
                       rotate: bool = True) -> dict:
    """Gather + statistics + transform + quantise the request's K/V (quant.py:483-695).

    Returns the same keys as the reference; `k8` / `vt8` are this build's tile images -- use
    `ws.k8_logical(n)` / `ws.v8_logical(n)` for position-order bytes.  `qk_i8` selects INT8 K bytes
    at amax/127 (the reference's default) instead of E4M3 at amax/448."""
    if need_vb16 or not need_vt8:
        raise ValueError("only the all-FP8-PV lane (need_vt8=True, need_vb16=False) is built")
    n, kvh = int(idx.shape[0]), int(k_buffer.shape[1])
    hq = ws.dims[2] if ws.dims and ws.dims[3] == kvh else max(kvh, DECLARED_Q_HEADS // DECLARED_KV_HEADS * kvh)
    ws.ensure(n, ws.dims[1] if ws.dims else 1, hq, kvh)
    lib = _kernel.load()
    call = make_call(ws, k_pool=k_buffer, v_pool=v_buffer, idx=idx, q_len=1, kv_len=n, prefix=0,
                     q_heads=hq, kv_heads=kvh, sm_scale=1.0, rotate=rotate, center_k=center_k, qk_i8=qk_i8)
    st = _stream(k_buffer.device)
    for fn in ("akl_kv_tile_stats", "akl_kv_means", "akl_kv_scales", "akl_kv_transform"):
        _kernel.check(getattr(lib, fn)(ctypes.byref(call), st), fn)
    nt = _ceil_to(n, BLK) // BLK
    return {"k8": ws.view("k8"), "kscale": ws.view("kscale")[:, :nt], "vt8": ws.view("v8t"),
            "vb16": None, "vscale": ws.view("vscale"), "vlog2r": ws.view("vlog2r")[:, :nt],
            "vinvr": ws.view("vinvr")[:, :nt], "vmean": ws.view("vmean"),
            "kmean": ws.view("kmean"), "vscale_t": ws.view("vst")[:, :nt], "n": n, "ntmax": nt}


def quantize_q(ws: FP8PrefillWorkspace, q, sm_scale: float, qk_i8: bool = True,
               rotate: bool = True):
    """-> (q8 tile images, qscale [H, Mpad] f32 per row with sm_scale folded, Mpad)
    (quant.py:433-480).  `qk_i8`: INT8 bytes at amax/127 instead of E4M3 at amax/448."""
    t, h = int(q.shape[0]), int(q.shape[1])
    kvh = ws.dims[3] if ws.dims and ws.dims[2] == h else DECLARED_KV_HEADS
    ws.ensure(ws.dims[0] if ws.dims else 1, t, h, kvh)
    lib = _kernel.load()
    # the pools are not read by this phase; any 16-byte-aligned device address satisfies the check
    call = make_call(ws, q=q, k_pool=q, v_pool=q, idx=q, q_len=t, kv_len=1, prefix=0, q_heads=h,
                     kv_heads=kvh, sm_scale=sm_scale, rotate=rotate, qk_i8=qk_i8)
    _kernel.check(lib.akl_quantize_q(ctypes.byref(call), _stream(q.device)), "akl_quantize_q")
    mpad = _ceil_to(t, MPAD)
    return ws.view("q8"), ws.view("qscale")[:, :mpad], mpad
