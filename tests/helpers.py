"""Comparison helpers shared by the GPU parity tests."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

import akl_oracle as O

#: measured parity figures, keyed "section/case/mode"; tests/conftest.py writes them to a
#: parity_ledger.json in the run's output folder when the session ends
LEDGER: dict = {}


def record(section: str, key: str, **metrics):
    LEDGER.setdefault(section, {})[key] = {k: (float(v) if isinstance(v, (float, np.floating)) else int(v)
                                               if isinstance(v, (int, np.integer, bool, np.bool_)) else v)
                                           for k, v in metrics.items()}


def max_over_rms(got: np.ndarray, ref: np.ndarray) -> float:
    """max|got - ref| / RMS(ref): the stated output metric."""
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    return float(np.abs(got.astype(np.float64) - ref).max() / max(rms, 1e-30))


LOG2E = np.float32(1.4426950408889634)
LOG2_448 = np.float32(8.807354922057604)


def fp8_extend(pkg, *args, **kw):
    """`prefill_extend` in the FP8-QK mode unless the caller names a mode (the operator's own
    default is the reference's: INT8 QK)."""
    kw.setdefault("qk_i8", False)
    return pkg.prefill_extend(*args, **kw)


def fp8_batch(pkg, *args, **kw):
    kw.setdefault("qk_i8", False)
    return pkg.prefill_extend_batch(*args, **kw)


def bf16_ulp(x: np.ndarray) -> np.ndarray:
    """Spacing of bfloat16 at |x| (8 significand bits)."""
    return np.exp2(np.floor(np.log2(np.maximum(np.abs(x), 2.0 ** -126))) - 7)


def output_within_bound(got: np.ndarray, ref: np.ndarray) -> np.ndarray:
    """Elementwise predicate |got - ref| <= 1e-2 * RMS(ref) + ulp_bf16(ref).

    The first term is the stated tolerance; the second is one quantum of the BF16 output
    type, without which no implementation -- the reference's own fp32 kernel arithmetic
    included -- can meet the bound on elements larger than ~2.5 RMS."""
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    return np.abs(got.astype(np.float64) - ref) <= 1e-2 * rms + bf16_ulp(ref)


def row_rel(got: np.ndarray, ref: np.ndarray) -> np.ndarray:
    """Row-relative L2 error per (row, head) vector (the reference's own metric,
    tests/kernel/test_oracle_a.py:175-181)."""
    d = (got.astype(np.float64) - ref).reshape(-1, ref.shape[-1])
    r = ref.astype(np.float64).reshape(-1, ref.shape[-1])
    return np.linalg.norm(d, axis=1) / np.maximum(np.linalg.norm(r, axis=1), 1e-30)


def to_dev(inp: dict, dev):
    return tuple(inp[k].to(dev) for k in ("q", "k_pool", "v_pool", "idx"))


def gathered(inp: dict):
    """(q, k, v) as float32 numpy in position order."""
    rows = inp["idx"].long()
    return (inp["q"].float().numpy(), inp["k_pool"][rows].float().numpy(),
            inp["v_pool"][rows].float().numpy())


def workspace_packs(ws, T: int, N: int, qk_i8: bool = False):
    """The kernel's own quantised artifacts as oracle packs (position-order bytes)."""
    nt = (N + 63) // 64
    mpad = (T + 127) // 128 * 128
    qp = O.QPack(q8=ws.q8_logical(T).cpu().numpy(),
                 qscale=ws.view("qscale")[:, :mpad].cpu().numpy(), mpad=mpad, qk_i8=qk_i8)
    kv = O.KVPack(
        k8=ws.k8_logical(N).cpu().numpy(), kscale=ws.view("kscale")[:, :nt].cpu().numpy(),
        kmean=ws.view("kmean").cpu().numpy(), v8=ws.v8_logical(N).cpu().numpy(),
        vst=ws.view("vst")[:, :nt].cpu().numpy(), vscale=ws.view("vscale").cpu().numpy(),
        vlog2r=ws.view("vlog2r")[:, :nt].cpu().numpy(), vinvr=ws.view("vinvr")[:, :nt].cpu().numpy(),
        vmean=ws.view("vmean").cpu().numpy(), n=N, qk_i8=qk_i8)
    return qp, kv


def run_phases(pkg, ws, q, kp, vp, idx, prefix, sm_scale, *, out=None, lse=None, rotate=True,
               center_k=True, dump=False, qk_i8=False):
    """Drive the phase entry points of the C ABI one by one (same work as akl_prefill_extend)."""
    from attn_kernel_lab_b200 import kernel as K, quant

    lib = K.load()
    T, H = int(q.shape[0]), int(q.shape[1])
    N, KVH = int(idx.numel()), int(kp.shape[1])
    ws.ensure(N, T, H, KVH)
    out = torch.empty_like(q) if out is None else out
    lse = torch.empty((T, H), dtype=torch.float32, device=q.device) if lse is None else lse
    call = quant.make_call(ws, q=q, k_pool=kp, v_pool=vp, idx=idx, out=out, lse_out=lse, q_len=T,
                           kv_len=N, prefix=prefix, q_heads=H, kv_heads=KVH, sm_scale=sm_scale,
                           rotate=rotate, center_k=center_k, qk_i8=qk_i8)
    st = torch.cuda.current_stream(q.device).cuda_stream
    for fn in ("akl_kv_tile_stats", "akl_quantize_q", "akl_kv_means", "akl_kv_scales",
               "akl_kv_transform"):
        K.check(getattr(lib, fn)(ctypes.byref(call), st), fn)
    dumps = None
    if dump:
        nt = (N + 63) // 64
        mt = (T + 127) // 128
        s_dump = torch.full((H, mt, nt, 128, 64), float("nan"), dtype=torch.float32, device=q.device)
        p_dump = torch.full((H, mt, nt, 128, 64), 0xAA, dtype=torch.uint8, device=q.device)
        K.check(lib.akl_attention_dump(ctypes.byref(call), s_dump.data_ptr(), p_dump.data_ptr(), st),
                "akl_attention_dump")
        dumps = (s_dump, p_dump)
    else:
        K.check(lib.akl_attention(ctypes.byref(call), st), "akl_attention")
    torch.cuda.synchronize()
    return out, lse, dumps


def kernel_softmax_restated(S_raw, qscale_rows, kscale, vlog2r, vinvr, prefix, row0, N, ntile):
    """The kernel's per-tile softmax arithmetic restated in numpy from the raw fp32 QK^T
    accumulators of one (head, 128-row tile): fp32 scale and running max, exp2 evaluated
    exactly.  Yields per tile (p_fp32 [128,64], alpha [128], m_new [128])."""
    m = np.full(128, -np.inf, np.float32)
    limit = np.minimum(prefix + row0 + np.arange(128), N - 1)
    for j in range(ntile):
        sc = (qscale_rows * kscale[j]).astype(np.float32)
        sv = (S_raw[j] * sc[:, None]).astype(np.float32)
        cols = j * 64 + np.arange(64)
        sv = np.where(cols[None, :] <= limit[:, None], sv, -np.inf).astype(np.float32)
        m_new = np.maximum(m, sv.max(axis=1))
        with np.errstate(invalid="ignore", over="ignore"):
            alpha = np.where(np.isneginf(m), 0, np.exp2(((m - m_new) * LOG2E).astype(np.float64))).astype(np.float32)
            pc = ((LOG2_448 + vlog2r[j]).astype(np.float32) - (m_new * LOG2E).astype(np.float32)).astype(np.float32)
            arg = (sv.astype(np.float64) * np.float64(LOG2E) + pc[:, None].astype(np.float64)).astype(np.float32)
            p = np.exp2(arg.astype(np.float64)).astype(np.float32)
        p = np.where(np.isfinite(sv), p, 0).astype(np.float32)
        yield j, p, alpha, m_new
        m = m_new


def oracle_row_block(q, k, v, prefix, sm_scale, head: int, kv_head: int, r0: int, r1: int, *, qk_i8=False,
                     rotation="butterfly", center_k=True):
    """The float64 oracle for query rows r0:r1 of one q head, from position-order CPU tensors
    q [T,H,256], k/v [N,KVH,256]: per-row Q quantisation and per-head K/V statistics are
    independent of the other rows and heads, so a block is exact, and cheap at any length.
    Returns (out [R,256] float32 bf16-rounded, lse [R] float32)."""
    qp, kv = oracle_block_packs(q, k, v, sm_scale, head, kv_head, r0, r1, qk_i8=qk_i8, rotation=rotation,
                                center_k=center_k)
    out, lse = O.attention(qp, kv, prefix + r0, r1 - r0, 1, return_lse=True)
    return out[:, 0], lse[:, 0]


def oracle_block_packs(q, k, v, sm_scale, head: int, kv_head: int, r0: int, r1: int, *, qk_i8=False,
                       rotation="butterfly", center_k=True):
    """Oracle packs for query rows r0:r1 of one q head and its KV head (see oracle_row_block);
    attend with prefix + r0 as the prefix and group 1."""
    qf = q[r0:r1, head:head + 1].float().numpy()
    kf = k[:, kv_head:kv_head + 1].float().numpy()
    vf = v[:, kv_head:kv_head + 1].float().numpy()
    qp = O.preprocess_q(qf, sm_scale, rotation=rotation, qk_i8=qk_i8)
    kv = O.preprocess_kv(kf, vf, rotation=rotation, center_k=center_k, qk_i8=qk_i8)
    return qp, kv


def assert_block_close(got_out, got_lse, ref_out, ref_lse, what=""):
    """Tolerance-level agreement of a row block with the oracle (quantised bytes equal up to rare
    one-code flips, so rows agree to rounding; a flipped P byte may move a peaked row more)."""
    rel = row_rel(got_out, ref_out)
    assert np.median(rel) < 2e-3 and (rel < 9e-3).mean() > 0.95, (what, float(np.median(rel)), float(rel.max()))
    fin = np.isfinite(ref_lse)
    assert np.array_equal(np.isfinite(got_lse), fin), what
    assert np.abs(got_lse[fin] - ref_lse[fin]).max() < 5e-3, what


def emulated_kv_split(pkg, q, kp, vp, idx, prefix, sm_scale, world, *, qk_i8=False):
    """The multi-GPU KV-axis split run as consecutive per-rank phase calls on ONE device (ranks
    that would wait on one another never share a GPU): tile sums per rank, the disjoint-support
    SUM, means per rank, the MAX of the raw V amax, then transform, Q and attention per rank, and
    the merge kernel.  Returns (merged_out, merged_lse, workspaces, ranges, outs, lses)."""
    from attn_kernel_lab_b200 import dist as D, kernel as K, quant

    lib = K.load()
    dev = q.device
    st = torch.cuda.current_stream(dev).cuda_stream
    T, Hq = int(q.shape[0]), int(q.shape[1])
    Hkv = int(kp.shape[1])
    n_total = int(idx.numel())
    ranges = D.kv_split_ranges(n_total, world)
    ntg = (n_total + 63) // 64
    wss = [pkg.FP8PrefillWorkspace(dev) for _ in ranges]
    calls, outs, lses = [], [], []
    slices = [idx[lo:hi].contiguous() for lo, hi in ranges]      # kept alive for the launches
    for ws, (lo, hi), part in zip(wss, ranges, slices):
        ws.ensure(n_total, T, Hq, Hkv)
        o = torch.empty_like(q)
        l = torch.empty((T, Hq), dtype=torch.float32, device=dev)
        c = quant.make_call(ws, q=q, k_pool=kp, v_pool=vp, idx=part, out=o, lse_out=l, q_len=T,
                            kv_len=hi - lo, prefix=prefix, q_heads=Hq, kv_heads=Hkv, sm_scale=sm_scale,
                            qk_i8=qk_i8, kv_pos0=lo, n_total=n_total, tile0_global=lo // 64,
                            ntiles_global=ntg)
        ws.view("ktsum")[:ntg].zero_()
        ws.view("vtsum")[:ntg].zero_()
        K.check(lib.akl_kv_tile_stats(ctypes.byref(c), st), "stats")
        calls.append(c), outs.append(o), lses.append(l)
    ksum = sum(ws.view("ktsum")[:ntg] for ws in wss)
    vsum = sum(ws.view("vtsum")[:ntg] for ws in wss)
    for ws, c in zip(wss, calls):
        ws.view("ktsum")[:ntg].copy_(ksum)
        ws.view("vtsum")[:ntg].copy_(vsum)
        K.check(lib.akl_kv_means(ctypes.byref(c), st), "means")
    vsmax = torch.stack([ws.view("vsmax") for ws in wss]).amax(dim=0)
    for ws, c in zip(wss, calls):
        ws.view("vsmax").copy_(vsmax)
        for fn in ("akl_kv_scales", "akl_kv_transform", "akl_quantize_q", "akl_attention"):
            K.check(getattr(lib, fn)(ctypes.byref(c), st), fn)
    merged, mlse = D.merge_states(outs, lses)
    torch.cuda.synchronize()
    assert all(ws.status() == 0 for ws in wss)
    del slices
    return merged, mlse, wss, ranges, outs, lses
