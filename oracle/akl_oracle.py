"""CPU oracle for the fused FP8 paged EXTEND/prefill attention operator.

THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the smoke
check and the benchmark's CPU-baseline leg may import it; the shipped operator
never calls into this file and has no CPU fallback.

It restates, in numpy with explicit float32 / float64 arithmetic, the algorithm
of the reference operator (sherkaner-underhill/attn-kernel-lab):

  * Q preprocessing        src/attn_kernel_lab/quant.py:433-480
                           (oracle form: src/attn_kernel_lab/oracle_a.py:105-116)
  * K/V statistics         src/attn_kernel_lab/quant.py:532-584
  * K transform            src/attn_kernel_lab/quant.py:589-611, :416-430
  * V transform            src/attn_kernel_lab/quant.py:613-635 (logical order, no SIGMA)
  * hygiene + fold arrays  src/attn_kernel_lab/quant.py:639-689
  * attention              src/attn_kernel_lab/oracle_a.py:211-286
  * split-KV composition   docs/OPERATOR_CONTRACT.md:238-242 (base-2 LSE merge)

Parity status: PINNED.  tests/test_oracle_golden.py checks every function here
against fixtures under tests/golden/ that were produced by importing and running
the reference's own Python (tests/golden/make_golden.py), and against the k8 /
vt8 sha256 digests of the reference's tests/kernel/golden_bitexact.json.

Two reductions of the reference have an order that belongs to the BLAS / tensor
library it runs on rather than to the operator (the fp32 rotation GEMM and the
fp32 channel sum).  For those this file offers both orders:

  rotation="sequential"  k = 0..255 accumulated in order in fp32; this is what the
                         reference's CPU GEMM does and reproduces its bytes.
  rotation="butterfly"   the fast Walsh-Hadamard order the CUDA kernels use
                         (stages h = 1, 2, 4, ..., 128, then an exact 1/16).
  means: `channel_sums_tiled` is the CUDA kernels' order (64-row tiles, eight
         8-row runs per tile, tiles added in order inside each 32768-row slab,
         slabs added in order).  The reference's own order is internal to its
         tensor library and cannot be restated; callers pin the rest of the
         pipeline by passing the reference's means in.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

HEAD_DIM = 256
BLK = 64          # quantisation tile along the kv axis (quant.py:80)
MPAD = 128        # query-row padding granule (quant.py:86)
SLAB = 32768      # normative statistics slab (quant.py:87)
FP8_MAX = 448.0
INT8_MAX = 127.0
F32 = np.float32


def ceil_to(x: int, m: int) -> int:
    return (x + m - 1) // m * m


# --------------------------------------------------------------------------
# number formats
# --------------------------------------------------------------------------

def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """uint16 bfloat16 bit patterns -> float32 (exact)."""
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns, round-to-nearest-even (NaN kept quiet)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    rounded = (u + (np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1)))) >> 16
    out = rounded.astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """float -> the float32 value of its bfloat16 rounding (via float32, as the
    reference's final `.to(torch.bfloat16)` does from float64)."""
    return bf16_bits_to_f32(f32_to_bf16_bits(np.asarray(x).astype(np.float32)))


_E4M3_TABLE = None


def e4m3_decode_table() -> np.ndarray:
    """All 256 E4M3 (fn variant: no inf, 0x7F/0xFF NaN) values as float32."""
    global _E4M3_TABLE
    if _E4M3_TABLE is None:
        t = np.zeros(256, dtype=np.float32)
        for b in range(256):
            s = -1.0 if b & 0x80 else 1.0
            e = (b >> 3) & 0xF
            m = b & 7
            if e == 0xF and m == 7:
                v = float("nan")
            elif e == 0:
                v = m * 2.0 ** -9
            else:
                v = (1.0 + m / 8.0) * 2.0 ** (e - 7)
            t[b] = s * v
        _E4M3_TABLE = t
    return _E4M3_TABLE


def e4m3_decode(b: np.ndarray) -> np.ndarray:
    return e4m3_decode_table()[np.asarray(b, dtype=np.uint8)]


def e4m3_encode(x: np.ndarray, overflow: str = "sat") -> np.ndarray:
    """float32 -> E4M3 byte, round-to-nearest-even, subnormals kept.

    overflow="sat": magnitudes above 448 clamp to 448 (the GPU's
    cvt.rn.satfinite).  overflow="nan": magnitudes that round past 448 become
    NaN (the tensor-library cast the reference calls normative,
    oracle_a.py:74-77).  The two agree wherever |x| <= 464, which is the whole
    domain of the operator (quotients are bounded by 448*(1+eps)).
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    a = np.abs(x).astype(np.float64)
    sign = np.signbit(x).astype(np.uint8) << 7
    _, ex = np.frexp(a)                      # a = m * 2**ex, m in [0.5, 1)
    e = np.maximum(ex - 1, -6)               # value exponent, floored at the subnormal one
    q = np.rint(np.ldexp(a, -(e - 3)))       # units of 2**(e-3); ties to even
    v = np.ldexp(q, e - 3)                   # rounded magnitude (may carry to next binade)
    over = v > 448.0
    v = np.minimum(v, 448.0)
    _, ex2 = np.frexp(v)
    e2 = ex2 - 1
    is_sub = v < 2.0 ** -6
    mant_sub = np.rint(v * 2.0 ** 9)
    mant_nrm = np.rint((np.ldexp(v, -np.where(is_sub, 0, e2)) - 1.0) * 8.0)
    byte = np.where(is_sub, mant_sub, ((e2 + 7) * 8) + mant_nrm).astype(np.int64)
    byte = np.where(v == 0, 0, byte)
    if overflow == "nan":
        byte = np.where(over, 0x7F, byte)
    byte = np.where(np.isnan(x), 0x7F, byte)
    return (byte.astype(np.uint8) | sign).astype(np.uint8)


# --------------------------------------------------------------------------
# rotation
# --------------------------------------------------------------------------

def hadamard(n: int = HEAD_DIM) -> np.ndarray:
    """Orthonormal Sylvester Hadamard matrix, H[i][j] = (-1)^popcount(i&j)/sqrt(n)
    (quant.py:107-112, oracle_a.py:59-66)."""
    h = np.ones((1, 1), dtype=np.float32)
    while h.shape[0] < n:
        h = np.block([[h, h], [h, -h]])
    return (h / F32(math.sqrt(n))).astype(np.float32)


def rotate_sequential(x: np.ndarray) -> np.ndarray:
    """x @ H in fp32 with k accumulated 0..255 in order.

    Every product x[k] * (+-1/16) is exact, so the result is a chain of 255
    rounded fp32 additions per output; this is the order the reference's CPU
    GEMM produces (quant.py:460-462, :600-601)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    lead = x.shape[:-1]
    xs = x.reshape(-1, HEAD_DIM) * F32(1.0 / 16.0)
    sign = (hadamard() * F32(16.0)).astype(np.float32)      # +-1
    acc = np.zeros_like(xs)
    for k in range(HEAD_DIM):
        acc = (acc + xs[:, k:k + 1] * sign[k:k + 1, :]).astype(np.float32)
    return acc.reshape(*lead, HEAD_DIM)


def rotate_butterfly(x: np.ndarray) -> np.ndarray:
    """x @ H evaluated as a fast Walsh-Hadamard transform in fp32.

    Stage order h = 1, 2, 4, ..., 128; each stage maps the pair (i, i+h) with
    bit h of i clear to (a + b, a - b); the result is multiplied by 1/16
    (exact).  This is the order of the CUDA transform kernels."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    lead = x.shape[:-1]
    y = x.reshape(-1, HEAD_DIM).copy()
    h = 1
    while h < HEAD_DIM:
        z = y.reshape(-1, HEAD_DIM // (2 * h), 2, h)
        a = z[:, :, 0, :]
        b = z[:, :, 1, :]
        y = np.stack([(a + b).astype(np.float32), (a - b).astype(np.float32)], axis=2)
        y = y.reshape(-1, HEAD_DIM)
        h *= 2
    return (y * F32(1.0 / 16.0)).astype(np.float32).reshape(*lead, HEAD_DIM)


def _rotate(x, rotation):
    if rotation == "sequential":
        return rotate_sequential(x)
    if rotation == "butterfly":
        return rotate_butterfly(x)
    if rotation in (None, "none", False):
        return np.ascontiguousarray(x, dtype=np.float32)
    raise ValueError(f"unknown rotation order {rotation!r}")


# --------------------------------------------------------------------------
# preprocessing
# --------------------------------------------------------------------------

@dataclass
class QPack:
    q8: np.ndarray        # [H, Mpad, D] uint8 (E4M3 bytes, or two's-complement INT8 when qk_i8)
    qscale: np.ndarray    # [H, Mpad] float32, sm_scale folded in
    mpad: int
    qk_i8: bool = False


@dataclass
class KVPack:
    k8: np.ndarray        # [KVH, Npad, D] uint8, position order
    kscale: np.ndarray    # [KVH, nt] float32
    kmean: np.ndarray     # [KVH, D] float32 (zeros when centring is off)
    v8: np.ndarray        # [KVH, Npad, D] uint8, position order (no SIGMA, no transpose)
    vst: np.ndarray       # [KVH, nt] float32: max(amax_t, vsmax/16)/448
    vscale: np.ndarray    # [KVH] float32: vsmax/448
    vlog2r: np.ndarray    # [KVH, nt] float32
    vinvr: np.ndarray     # [KVH, nt] float32
    vmean: np.ndarray     # [KVH, D] float32
    n: int
    qk_i8: bool = False   # K bytes are two's-complement INT8 at scale amax/127 (V stays E4M3)


def qk_quantise(x: np.ndarray, scale: np.ndarray, qk_i8: bool) -> np.ndarray:
    """Q/K bytes of one scale group (quant.py:416-430, 471-478): E4M3 of the IEEE quotient, or
    for INT8 the quotient rounded half-to-even and stored as two's complement, without a clamp
    (|x| <= amax bounds the quotient at 127 (1 + 2 eps))."""
    quo = (x / scale).astype(np.float32)
    if qk_i8:
        return np.rint(quo).astype(np.int8).view(np.uint8)
    return e4m3_encode(quo)


def qk_decode(b: np.ndarray, qk_i8: bool) -> np.ndarray:
    """float64 values of Q/K bytes."""
    if qk_i8:
        return np.asarray(b, np.uint8).view(np.int8).astype(np.float64)
    return e4m3_decode_table().astype(np.float64)[np.asarray(b, np.uint8)]


def preprocess_q(q: np.ndarray, sm_scale: float, rotation="butterfly", qk_i8: bool = False) -> QPack:
    """q [T, H, D] float32 (bf16-valued) -> QPack (quant.py:455-480).

    Rotate; zero-pad rows to a multiple of 128; per-row amax clamped at 1e-8;
    scale = amax / lim (IEEE division; lim 448 for E4M3, 127 for INT8); bytes =
    quantise(x / scale); exported scale = scale * sm_scale."""
    T, H, D = q.shape
    mpad = ceil_to(T, MPAD)
    qf = np.transpose(np.asarray(q, dtype=np.float32), (1, 0, 2))
    qf = _rotate(qf, rotation)
    if mpad != T:
        qf = np.concatenate([qf, np.zeros((H, mpad - T, D), np.float32)], axis=1)
    amax = np.maximum(qf.max(axis=2), -qf.min(axis=2)).astype(np.float32)
    amax = np.maximum(amax, F32(1e-8))
    scale = (amax / F32(INT8_MAX if qk_i8 else FP8_MAX)).astype(np.float32)
    q8 = qk_quantise(qf, scale[:, :, None], qk_i8)
    return QPack(q8=q8, qscale=(scale * F32(sm_scale)).astype(np.float32), mpad=mpad, qk_i8=qk_i8)


def channel_sums_tiled(x: np.ndarray, slab: int = SLAB) -> np.ndarray:
    """fp32 channel sums of x [N, KVH, D] in the CUDA kernels' order.

    Each 64-row tile is cut into eight runs of 8 consecutive rows; a run is
    summed row by row starting from +0; the eight run sums are added in order
    (again from +0); tile sums are added in order inside each `slab`-row slab
    (slab-by-slab accumulation is the reference's normative grouping,
    quant.py:543-568 and docs/OPERATOR_CONTRACT.md section 3); slab sums are
    added in order."""
    x = np.asarray(x, dtype=np.float32)
    N, KVH, D = x.shape
    npad = ceil_to(max(N, 1), BLK)
    xp = np.zeros((npad, KVH, D), np.float32)
    xp[:N] = x                                      # +0 rows: x + 0 == x exactly
    runs = xp.reshape(npad // 8, 8, KVH, D)
    run_sum = np.zeros((npad // 8, KVH, D), np.float32)
    for i in range(8):
        run_sum = (run_sum + runs[:, i]).astype(np.float32)
    per_tile = run_sum.reshape(npad // BLK, 8, KVH, D)
    tile_sum = np.zeros((npad // BLK, KVH, D), np.float32)
    for w in range(8):
        tile_sum = (tile_sum + per_tile[:, w]).astype(np.float32)
    total = np.zeros((KVH, D), np.float32)
    tiles_per_slab = slab // BLK
    for s0 in range(0, npad // BLK, tiles_per_slab):
        slab_sum = np.zeros((KVH, D), np.float32)
        for t in range(s0, min(s0 + tiles_per_slab, npad // BLK)):
            slab_sum = (slab_sum + tile_sum[t]).astype(np.float32)
        total = (total + slab_sum).astype(np.float32)
    return total


def preprocess_kv(
    k: np.ndarray,                 # [N, KVH, D] float32 (bf16/fp16-valued), position order
    v: np.ndarray,
    rotation="butterfly",
    center_k: bool = True,
    kmean: np.ndarray | None = None,
    vmean: np.ndarray | None = None,
    vsmax_raw: np.ndarray | None = None,
    qk_i8: bool = False,
) -> KVPack:
    """Statistics, K transform, V transform and fold arrays (quant.py:483-695).

    `kmean` / `vmean` override the channel means (used to pin every later step
    against the reference, whose mean reduction order cannot be restated, and to
    hand a KV-axis split the request-wide means).  `vsmax_raw` overrides the
    per-head maximum of the centred per-tile V amax (request-wide for a split).
    The raw maximum this slice would have produced is stored on the result as
    `vsmax_local`."""
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    N, KVH, D = k.shape
    npad = ceil_to(N, BLK)
    nt = npad // BLK
    denom = F32(max(N, 1))

    # ---- statistics (quant.py:532-584)
    if vmean is None:
        vmean = (channel_sums_tiled(v) / denom).astype(np.float32)
    if center_k:
        if kmean is None:
            kmean = (channel_sums_tiled(k) / denom).astype(np.float32)
    else:
        kmean = np.zeros((KVH, D), np.float32)
    vh = np.transpose(v, (1, 0, 2))                              # [KVH, N, D]
    vtmx = np.full((KVH, nt, D), -np.inf, np.float32)
    vtmn = np.full((KVH, nt, D), np.inf, np.float32)
    for t in range(nt):
        rows = vh[:, t * BLK:min((t + 1) * BLK, N)]               # real rows only
        vtmx[:, t] = rows.max(axis=1)
        vtmn[:, t] = rows.min(axis=1)
    vam = np.maximum((vtmx - vmean[:, None, :]).astype(np.float32),
                     (vmean[:, None, :] - vtmn).astype(np.float32)).max(axis=2)
    vsmax_local = vam.max(axis=1).astype(np.float32)
    vsmax = np.maximum(vsmax_local if vsmax_raw is None else np.asarray(vsmax_raw, np.float32),
                       F32(1e-8)).astype(np.float32)
    vst = (np.maximum(vam, (vsmax[:, None] / F32(16.0)).astype(np.float32))
           / F32(FP8_MAX)).astype(np.float32)

    # ---- K (quant.py:589-611): centre, rotate, pad with zeros, per-tile amax, quantise
    kh = np.transpose(k, (1, 0, 2))
    kf = (kh - kmean[:, None, :]).astype(np.float32) if center_k else kh.astype(np.float32)
    kf = _rotate(kf, rotation)
    if npad != N:
        kf = np.concatenate([kf, np.zeros((KVH, npad - N, D), np.float32)], axis=1)
    kb = kf.reshape(KVH, nt, BLK * D)
    kam = np.maximum(np.maximum(kb.max(axis=2), -kb.min(axis=2)), F32(1e-8)).astype(np.float32)
    kscale = (kam / F32(INT8_MAX if qk_i8 else FP8_MAX)).astype(np.float32)
    k8 = qk_quantise(kf.reshape(KVH, nt, BLK, D), kscale[:, :, None, None], qk_i8)
    k8 = k8.reshape(KVH, npad, D)

    # ---- V (quant.py:613-635): centre, pad with zeros, per-tile scale, quantise
    vf = (vh - vmean[:, None, :]).astype(np.float32)
    if npad != N:
        vf = np.concatenate([vf, np.zeros((KVH, npad - N, D), np.float32)], axis=1)
    v8 = e4m3_encode((vf.reshape(KVH, nt, BLK, D) / vst[:, :, None, None]).astype(np.float32))
    v8 = v8.reshape(KVH, npad, D)

    # ---- fold arrays (quant.py:673-679)
    r = ((vst * F32(FP8_MAX)).astype(np.float32) / vsmax[:, None]).astype(np.float32)
    r = np.clip(r, F32(1.0 / 16.0), F32(1.0)).astype(np.float32)
    vlog2r = np.log2(r).astype(np.float32)
    vinvr = (F32(1.0) / r).astype(np.float32)
    vscale = (vsmax / F32(FP8_MAX)).astype(np.float32)
    pack = KVPack(k8=k8, kscale=kscale, kmean=kmean, v8=v8, vst=vst, vscale=vscale,
                  vlog2r=vlog2r, vinvr=vinvr, vmean=vmean, n=N, qk_i8=qk_i8)
    pack.vsmax_local = vsmax_local
    return pack


# --------------------------------------------------------------------------
# the operator (oracle_a.py:211-286), vectorised over query rows
# --------------------------------------------------------------------------

def attention(
    qp: QPack,
    kv: KVPack,
    prefix: int,
    T: int,
    group: int,
    return_lse: bool = False,
    heads=None,
    kv_lo: int = 0,
    kv_hi: int | None = None,
    collect_p: dict | None = None,
):
    """The intended quantised operator in float64.

    Row r sees columns 0 .. min(prefix + r, n - 1).  Per 64-column tile, in
    order: dequantised scores; running max; P rounded to E4M3 at scale
    448*r_t; PV accumulates the rounded P against the stored V bytes; l
    accumulates the unrounded p*448; epilogue multiplies vscale/l and adds the
    V mean.  Returns bf16-rounded float32 [T, H_sel, D] (and base-2 LSE
    [T, H_sel] float32).

    `heads` selects a subset of query heads (default all).  `kv_lo:kv_hi`
    (multiples of 64) restricts the tiles visited -- the per-split operator of a
    KV-axis split; statistics inside `kv` stay global.  `collect_p`, when a dict, receives
    the E4M3 P bytes of every visited tile as collect_p[(head, tile)] = uint8 [T, width]."""
    H = qp.q8.shape[0]
    KVH, npad, D = kv.k8.shape
    n = kv.n
    heads = list(range(H)) if heads is None else list(heads)
    kv_hi = n if kv_hi is None else min(kv_hi, n)
    assert kv_lo % BLK == 0
    dec = e4m3_decode_table().astype(np.float64)
    out = np.zeros((T, len(heads), D), np.float32)
    lse = np.full((T, len(heads)), -np.inf, np.float32)
    rows = np.arange(T)
    vis_end = np.minimum(prefix + rows + 1, kv_hi)            # exclusive visible end per row
    for hi_, h in enumerate(heads):
        kvh = h // group
        qf = qk_decode(qp.q8[h, :T], qp.qk_i8)                # [T, D]
        qs = qp.qscale[h, :T].astype(np.float64)
        m = np.full(T, -np.inf)
        l = np.zeros(T)
        acc = np.zeros((T, D))
        last = int((vis_end.max() - 1) // BLK) if vis_end.max() > kv_lo else -1
        for t in range(kv_lo // BLK, last + 1):
            lo = t * BLK
            width = min(lo + BLK, n) - lo
            kf = qk_decode(kv.k8[kvh, lo:lo + width], kv.qk_i8)   # [w, D]
            s = (qf @ kf.T) * qs[:, None] * float(kv.kscale[kvh, t])
            cols = lo + np.arange(width)
            visible = cols[None, :] < vis_end[:, None]
            s = np.where(visible, s, -np.inf)
            tile_max = s.max(axis=1)
            m_new = np.maximum(m, tile_max)
            with np.errstate(invalid="ignore"):
                alpha = np.where(np.isneginf(m), 0.0, np.exp(m - m_new))
                p = np.where(visible, np.exp(s - m_new[:, None]), 0.0)
            alpha = np.where(np.isneginf(m_new), 1.0, alpha)   # row not started yet
            r_t = 1.0 / float(kv.vinvr[kvh, t])
            p8_bytes = e4m3_encode((p * (FP8_MAX * r_t)).astype(np.float32))
            if collect_p is not None:
                collect_p[(h, t)] = p8_bytes
            p8 = dec[p8_bytes]
            vf = dec[kv.v8[kvh, lo:lo + width]]
            acc = acc * alpha[:, None] + p8 @ vf
            l = l * alpha + p.sum(axis=1) * FP8_MAX
            m = m_new
        with np.errstate(divide="ignore", invalid="ignore"):
            inv_l = np.where(l > 0, float(kv.vscale[kvh]) / l, 0.0)
            o = acc * inv_l[:, None] + kv.vmean[kvh].astype(np.float64)[None, :]
            out[:, hi_] = round_to_bf16(o)
            lse[:, hi_] = np.where(
                l > 0, m / math.log(2.0) + np.log2(l) - math.log2(FP8_MAX), -np.inf
            ).astype(np.float32)
    return (out, lse) if return_lse else out


def merge_splits(outs, lses):
    """Combine per-split (O_i, lse2_i) into the whole-row result in float64.

    lse = log2(sum_i 2^lse_i); O = sum_i 2^(lse_i - lse) * O_i.  Each O_i already
    carries the V mean, and the weights sum to one, so the mean is counted once
    (docs/OPERATOR_CONTRACT.md:238-242).  Splits in which a row saw no key carry
    lse_i = -inf and weight 0."""
    lses = np.stack([np.asarray(x, np.float64) for x in lses])            # [S, T, H]
    outs = np.stack([np.asarray(x, np.float64) for x in outs])            # [S, T, H, D]
    mx = lses.max(axis=0)
    safe = np.where(np.isneginf(mx), 0.0, mx)
    w = np.exp2(lses - safe[None])
    den = w.sum(axis=0)
    with np.errstate(divide="ignore", invalid="ignore"):
        lse = np.where(den > 0, safe + np.log2(den), -np.inf)
        o = (w[..., None] * np.where(w[..., None] > 0, outs, 0.0)).sum(axis=0) / np.where(den > 0, den, 1.0)[..., None]
    return round_to_bf16(o), lse.astype(np.float32)


def reference(q, k, v, prefix, sm_scale=None, return_lse=False, rotation="butterfly",
              center_k=True, heads=None, qk_i8=False):
    """Whole pipeline from bf16-valued float32 inputs (oracle_a.py:289-301; `qk_i8` selects the
    reference's INT8-QK default, otherwise the FP8-QK form)."""
    T, H, D = q.shape
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    qp = preprocess_q(q, sm_scale, rotation=rotation, qk_i8=qk_i8)
    kv = preprocess_kv(k, v, rotation=rotation, center_k=center_k, qk_i8=qk_i8)
    return attention(qp, kv, prefix, T, group=H // k.shape[1], return_lse=return_lse, heads=heads)


# --------------------------------------------------------------------------
# fp32 plain attention (no quantisation) -- a gross-error yardstick only
# --------------------------------------------------------------------------

def plain_attention(q, k, v, prefix, sm_scale):
    """Unquantised bottom-right-causal GQA attention in float64 (explicit mask)."""
    T, H, D = q.shape
    N, KVH, _ = k.shape
    g = H // KVH
    out = np.zeros((T, H, D))
    cols = np.arange(N)[None, :]
    vis = cols <= (prefix + np.arange(T))[:, None]
    for h in range(H):
        s = (q[:, h].astype(np.float64) @ k[:, h // g].astype(np.float64).T) * sm_scale
        s = np.where(vis, s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, h] = (p / p.sum(axis=1, keepdims=True)) @ v[:, h // g].astype(np.float64)
    return out
