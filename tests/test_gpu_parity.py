"""Parity of the CUDA path (called through the C ABI) against the CPU oracle, on a B200.

Bars, as stated where they are asserted:
  * quantised Q/K/V bytes, scales, means, fold arrays: BIT-EXACT against the oracle evaluated
    in the kernels' documented reduction order (log2 of the fold ratio: last place);
  * raw QK^T accumulators: equal to the exact integer-like dot product to fp32 rounding;
  * P bytes: equal to the kernel's formula evaluated with an exact exp2, up to rare one-code
    flips from the approximate ex2 unit;
  * BF16 output: |d| <= 1e-2 * RMS(O_ref) + ulp_bf16(O_ref) against (a) float64 PV over the
    kernel's own P bytes, every element, and (b) the independent float64 oracle on every row
    whose P bytes agree with the oracle's; rows with a flipped P byte are counted and bounded;
  * base-2 LSE: |d| < 5e-3 (the reference's bound, tests/kernel/test_oracle_a.py:224-228).
"""
import ctypes
import hashlib
import json
import pathlib

import numpy as np
import pytest
import torch

import akl_oracle as O
import cases
import helpers as H

pytestmark = pytest.mark.gpu
GOLDEN = pathlib.Path(__file__).resolve().parent / "golden"
DIGESTS = json.loads((GOLDEN / "bitexact_digests.json").read_text())["cases"]
DIGESTS_I8 = json.loads((GOLDEN / "bitexact_digests.json").read_text())["cases_i8"]
SIGMA32 = [0, 1, 8, 9, 2, 3, 10, 11, 4, 5, 12, 13, 6, 7, 14, 15,
           16, 17, 24, 25, 18, 19, 26, 27, 20, 21, 28, 29, 22, 23, 30, 31]
SIGMA64 = [(j // 32) * 32 + SIGMA32[j % 32] for j in range(64)]

EXTRA_CASES = [
    cases._case("three_qtiles_300_1500", 300, 1500, 1200, 24, 4, "scattered", "outlier", 4401),
    cases._case("prefix0_257_257", 257, 257, 0, 16, 4, "contiguous", "jitter", 4402),
    cases._case("one_row_1_1", 1, 1, 0, 16, 4, "contiguous", "uniform", 4403),
    cases._case("one_row_deep_1_1000", 1, 1000, 999, 32, 4, "scattered", "outlier", 4404),
    cases._case("odd_tiles_64_192", 64, 192, 128, 24, 4, "scattered", "uniform", 4405, rotate=False, center_k=False),
]
ALL_CASES = cases.GOLDEN_CASES + EXTRA_CASES


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def gen_cap(pkg, case):
    return pkg.V1_CAPABILITY if (case["H"], case["KVH"]) in ((16, 4), (24, 4), (32, 4)) else pkg.GENERALIZATION_CAPABILITY


def assert_prep_exact(ws, qp, kv, T, N):
    nt = (N + 63) // 64
    mpad = (T + 127) // 128 * 128
    assert np.array_equal(bits(ws.view("kmean").cpu().numpy()), bits(kv.kmean)), "kmean"
    assert np.array_equal(bits(ws.view("vmean").cpu().numpy()), bits(kv.vmean)), "vmean"
    if qp is not None:
        assert np.array_equal(ws.q8_logical(T).cpu().numpy(), qp.q8), "q8"
        assert np.array_equal(bits(ws.view("qscale")[:, :mpad].cpu().numpy()), bits(qp.qscale)), "qscale"
    assert np.array_equal(ws.k8_logical(N).cpu().numpy(), kv.k8), "k8"
    assert np.array_equal(ws.v8_logical(N).cpu().numpy(), kv.v8), "v8"
    for name, ref in (("kscale", kv.kscale), ("vst", kv.vst), ("vinvr", kv.vinvr)):
        assert np.array_equal(bits(ws.view(name)[:, :nt].cpu().numpy()), bits(ref)), name
    assert np.array_equal(bits(ws.view("vscale").cpu().numpy()), bits(kv.vscale)), "vscale"
    assert np.abs(ws.view("vlog2r")[:, :nt].cpu().numpy() - kv.vlog2r).max() <= 2.4e-7, "vlog2r"


# ------------------------------------------------------------------ preprocessing
QK_MODES = pytest.mark.parametrize("qk_i8", [False, True], ids=["qk_fp8", "qk_int8"])


@QK_MODES
@pytest.mark.parametrize("case", ALL_CASES, ids=lambda c: c["name"])
def test_preprocessing_is_bit_exact(pkg, cuda, case, qk_i8):
    inp = cases.make_inputs(case)
    q, kp, vp, idx = H.to_dev(inp, cuda)
    ws = pkg.FP8PrefillWorkspace(cuda)
    H.run_phases(pkg, ws, q, kp, vp, idx, case["prefix"], case["sm_scale"], rotate=case["rotate"],
                 center_k=case["center_k"], qk_i8=qk_i8)
    qf, kf, vf = H.gathered(inp)
    rot = "butterfly" if case["rotate"] else None
    qp = O.preprocess_q(qf, case["sm_scale"], rotation=rot, qk_i8=qk_i8)
    kv = O.preprocess_kv(kf, vf, rotation=rot, center_k=case["center_k"], qk_i8=qk_i8)
    assert_prep_exact(ws, qp, kv, case["T"], case["N"])
    assert ws.status() == 0


def test_preprocessing_across_statistics_slabs(pkg, cuda):
    """More than two 32768-row slabs: tile sums are added inside a slab, then slabs are added
    (the reference pins the slab grouping, docs/OPERATOR_CONTRACT.md section 3.3)."""
    g = torch.Generator().manual_seed(4501)
    n, kvh = 70_001, 4
    k = (torch.randn(n, kvh, 256, generator=g) + 0.5).to(torch.bfloat16)
    v = (torch.randn(n, kvh, 256, generator=g) * 2 - 0.25).to(torch.bfloat16)
    idx = torch.randperm(n, generator=g)
    ws = pkg.FP8PrefillWorkspace(cuda)
    from attn_kernel_lab_b200 import quant

    kvd = quant.gather_quantize_kv(ws, k.to(cuda), v.to(cuda), idx.to(cuda), qk_i8=False)
    torch.cuda.synchronize()
    assert kvd["n"] == n and kvd["ntmax"] == (n + 63) // 64
    kv = O.preprocess_kv(k[idx].float().numpy(), v[idx].float().numpy())
    assert_prep_exact(ws, None, kv, 1, n)


@pytest.mark.parametrize("cid", sorted(DIGESTS), ids=lambda s: s.replace("|", "-"))
def test_reference_golden_digests_on_the_gpu(pkg, cuda, cid):
    """The reference's own sha256 goldens (tests/kernel/golden_bitexact.json, FP8-QK cases):
    V bytes in every case, K bytes wherever no rotation GEMM is involved."""
    meta, arts = DIGESTS[cid]["meta"], DIGESTS[cid]["artifacts"]
    inp = cases.bitexact_inputs(meta)
    q, kp, vp, idx = H.to_dev(inp, cuda)
    ws = pkg.FP8PrefillWorkspace(cuda)
    H.run_phases(pkg, ws, q, kp, vp, idx, meta["prefix"], 1.0 / 16.0, rotate=meta["rotate"],
                 center_k=meta["center_k"])
    v8 = ws.v8_logical(meta["N"]).cpu().numpy()
    kvh, npad, d = v8.shape
    vt8 = v8.reshape(kvh, npad // 64, 64, d)[:, :, SIGMA64, :].transpose(0, 1, 3, 2)
    assert sha(vt8) == arts["vt8"]
    if not meta["rotate"]:
        assert sha(ws.k8_logical(meta["N"]).cpu().numpy()) == arts["k8"]


@pytest.mark.parametrize("cid", sorted(DIGESTS_I8), ids=lambda s: s.replace("|", "-"))
def test_reference_golden_digests_int8_qk_on_the_gpu(pkg, cuda, cid):
    """The INT8-QK cases of the same matrix: V bytes in every case; K and Q bytes wherever no
    rotation GEMM is involved (there the arithmetic is the same division and rounding)."""
    meta, arts = DIGESTS_I8[cid]["meta"], DIGESTS_I8[cid]["artifacts"]
    inp = cases.bitexact_inputs(meta)
    q, kp, vp, idx = H.to_dev(inp, cuda)
    ws = pkg.FP8PrefillWorkspace(cuda)
    H.run_phases(pkg, ws, q, kp, vp, idx, meta["prefix"], 1.0 / 16.0, rotate=meta["rotate"],
                 center_k=meta["center_k"], qk_i8=True)
    v8 = ws.v8_logical(meta["N"]).cpu().numpy()
    kvh, npad, d = v8.shape
    vt8 = v8.reshape(kvh, npad // 64, 64, d)[:, :, SIGMA64, :].transpose(0, 1, 3, 2)
    assert sha(vt8) == arts["vt8"]
    if not meta["rotate"]:
        assert sha(ws.k8_logical(meta["N"]).cpu().numpy()) == arts["k8"]
        assert sha(ws.q8_logical(meta["T"]).cpu().numpy()[:, :meta["T"]]) == arts["q8"]


# ------------------------------------------------------------------ attention
@QK_MODES
@pytest.mark.parametrize("case", ALL_CASES, ids=lambda c: c["name"])
def test_attention_scores_probabilities_and_output(pkg, cuda, case, qk_i8):
    T, N, Hq, KVH, prefix = case["T"], case["N"], case["H"], case["KVH"], case["prefix"]
    g = Hq // KVH
    inp = cases.make_inputs(case)
    q, kp, vp, idx = H.to_dev(inp, cuda)
    ws = pkg.FP8PrefillWorkspace(cuda)
    out, lse, (s_dump, p_dump) = H.run_phases(pkg, ws, q, kp, vp, idx, prefix, case["sm_scale"],
                                              rotate=case["rotate"], center_k=case["center_k"], dump=True,
                                              qk_i8=qk_i8)
    assert ws.status() == 0
    qp, kv = H.workspace_packs(ws, T, N, qk_i8)
    sd, pd = s_dump.cpu().numpy(), p_dump.cpu().numpy()
    got, got_lse = out.float().cpu().numpy(), lse.cpu().numpy()
    dec = O.e4m3_decode_table().astype(np.float64)
    nt, mt = (N + 63) // 64, (T + 127) // 128

    own = np.zeros((T, Hq, 256), np.float32)            # float64 PV over the kernel's own P bytes
    flips_formula = total_p = 0
    for h in range(Hq):
        kvh = h // g
        S = O.qk_decode(qp.q8[h], qk_i8) @ O.qk_decode(kv.k8[kvh], qk_i8).T   # exact: every partial sum fits a double
        for qt in range(mt):
            hi = min(prefix + qt * 128 + 128, N)
            ntile = (hi + 63) // 64
            for j in range(ntile):                      # raw accumulators
                ref = S[qt * 128:(qt + 1) * 128, j * 64:(j + 1) * 64]
                err = np.abs(sd[h, qt, j][:, :ref.shape[1]] - ref).max()
                assert err <= (0.0 if qk_i8 else 2e-6 * max(1.0, np.abs(ref).max())), "QK^T accumulators"
            l = np.zeros(128, np.float32)
            acc = np.zeros((128, 256))
            m = None
            for j, p, alpha, m in H.kernel_softmax_restated(
                    sd[h, qt], qp.qscale[h, qt * 128:(qt + 1) * 128], kv.kscale[kvh], kv.vlog2r[kvh],
                    kv.vinvr[kvh], prefix, qt * 128, N, ntile):
                want8 = O.e4m3_encode(p)
                ne = want8 != pd[h, qt, j]
                flips_formula += int(ne.sum())
                total_p += ne.size
                if ne.any():
                    assert np.abs(want8.astype(np.int16) - pd[h, qt, j].astype(np.int16))[ne].max() == 1
                cols = j * 64 + np.arange(64)
                lim = np.minimum(prefix + qt * 128 + np.arange(128), N - 1)
                assert not pd[h, qt, j][cols[None, :] > lim[:, None]].any(), "masked P must be exact zeros"
                l = (l * alpha + p.sum(axis=1) * kv.vinvr[kvh, j]).astype(np.float32)
                vt = np.zeros((64, 256))
                nn = min(64, N - j * 64)
                vt[:nn] = dec[kv.v8[kvh, j * 64:j * 64 + nn]]
                acc = acc * alpha[:, None].astype(np.float64) + dec[pd[h, qt, j]] @ vt
            inv = np.where(l > 0, kv.vscale[kvh] / l, 0)
            o = O.round_to_bf16(acc * inv[:, None] + kv.vmean[kvh][None, :])
            r0, r1 = qt * 128, min(T, qt * 128 + 128)
            own[r0:r1, h] = o[:r1 - r0]
    assert flips_formula <= max(2, 2e-5 * total_p), f"P flips vs exact exp2: {flips_formula}/{total_p}"
    assert H.output_within_bound(got, own).all(), "output vs float64 PV over the kernel's own P"
    assert (got != own).mean() < 5e-3
    ledger = {"p_flips_vs_exact_exp2": flips_formula, "p_bytes": total_p,
              "max_over_rms_vs_f64_pv_of_own_p": H.max_over_rms(got, own),
              "bf16_elements_differing_from_f64_pv": float((got != own).mean())}

    # the independent float64 oracle, on the kernel's own quantised bytes (the reference's
    # pattern, tests/kernel/test_ops_gpu.py:48-68)
    their_p = {}
    ref, ref_lse = O.attention(qp, kv, prefix, T, g, return_lse=True, collect_p=their_p)
    assert np.abs(got_lse - ref_lse).max() < 5e-3
    flipped = np.zeros((T, Hq), bool)
    for (h, t), p8 in their_p.items():
        for qt in range(mt):
            r0, r1 = qt * 128, min(T, qt * 128 + 128)
            hi = min(prefix + qt * 128 + 128, N)
            if t >= (hi + 63) // 64:
                continue
            mine = pd[h, qt, t][:r1 - r0, :p8.shape[1]]
            flipped[r0:r1, h] |= (mine != p8[r0:r1]).any(axis=1)
    ok = H.output_within_bound(got, ref)
    assert ok[~flipped].all(), "rows whose P bytes equal the oracle's must meet the output bound"
    assert flipped.sum() <= max(2, 0.01 * flipped.size), f"{flipped.mean():.3%} of rows carry a P flip"   # observed: at most 0.4 %
    rel = H.row_rel(got, ref).reshape(T, Hq)
    assert (rel[~flipped] < 9e-3).all() if (~flipped).any() else True
    assert (rel >= 9e-3).sum() <= max(1, 0.002 * rel.size), "rows over the reference's own row-relative bound"   # observed: one row in one case
    ledger.update({"rows": int(flipped.size), "rows_with_a_p_flip_vs_oracle": int(flipped.sum()),
                   "max_over_rms_vs_oracle_all_rows": H.max_over_rms(got, ref),
                   "max_over_rms_vs_oracle_unflipped_rows": (H.max_over_rms(got[~flipped], ref[~flipped]) if (~flipped).any() else 0.0),
                   "rows_over_9e-3": int((rel >= 9e-3).sum()), "rowrel_median": float(np.median(rel)),
                   "rowrel_max": float(rel.max()), "lse_max_abs": float(np.abs(got_lse - ref_lse).max())})
    H.record("attention_vs_oracle", f"{case['name']}/{'int8' if qk_i8 else 'fp8'}", **ledger)


# ------------------------------------------------------------------ the public operator
def _public(pkg, cuda, case, **kw):
    inp = cases.make_inputs(case)
    q, kp, vp, idx = H.to_dev(inp, cuda)
    return inp, (q, kp, vp, idx), H.fp8_extend(pkg, 
        q, kp, vp, idx, case["prefix"], sm_scale=case["sm_scale"], rotate=case["rotate"],
        center_k=case["center_k"], capability=gen_cap(pkg, case), **kw)


def test_public_entry_equals_the_phase_calls_and_honours_out(pkg, cuda):
    case = cases.GOLDEN_CASES[0]
    inp, (q, kp, vp, idx), (out, lse) = _public(pkg, cuda, case, return_lse=True)
    ws = pkg.FP8PrefillWorkspace(cuda)
    out2, lse2, _ = H.run_phases(pkg, ws, q, kp, vp, idx, case["prefix"], case["sm_scale"])
    assert torch.equal(out, out2) and torch.equal(lse, lse2)
    mine = torch.full_like(q, float("nan"))
    mine_lse = torch.full((case["T"], case["H"]), float("nan"), device=cuda)
    res = H.fp8_extend(pkg, q, kp, vp, idx, case["prefix"], sm_scale=case["sm_scale"], out=mine,
                             lse_out=mine_lse, return_lse=True)
    assert res[0] is mine and res[1] is mine_lse and torch.equal(mine, out) and torch.equal(mine_lse, lse)
    only = H.fp8_extend(pkg, q, kp, vp, idx, case["prefix"], sm_scale=case["sm_scale"])
    assert isinstance(only, torch.Tensor) and torch.equal(only, out)      # LSE request does not move O
    assert out.shape == q.shape and out.dtype == torch.bfloat16 and lse.dtype == torch.float32


def test_against_the_reference_output_fixture(pkg, cuda):
    """Benchmark configuration 1 end to end against the output the reference's own oracle
    produced (tests/golden/c1_cpu_oracle.npz): the kernels' reduction order differs from the
    reference's CPU library in the last place of a few means/scales, so this is the
    tolerance-level check (row-relative L2, the reference's own metric)."""
    case = cases.GOLDEN_CASES[0]
    g = np.load(GOLDEN / "c1_cpu_oracle.npz")
    _, _, (out, lse) = _public(pkg, cuda, case, return_lse=True)
    heads = g["heads"].tolist()
    ref = O.bf16_bits_to_f32(g["out_bf16_bits"])
    got = out.float().cpu().numpy()[:, heads]
    rel = H.row_rel(got, ref)
    H.record("public_entry_vs_reference_output_fixture", "c1_cpu_oracle/fp8", rowrel_median=float(np.median(rel)),
             rowrel_max=float(rel.max()), rows_over_9e_3=int((rel >= 9e-3).sum()), rows=int(rel.size),
             max_over_rms=H.max_over_rms(got, ref), lse_max_abs=float(np.abs(lse.cpu().numpy()[:, heads] - g["lse"]).max()))
    assert np.median(rel) < 2e-3 and (rel < 9e-3).mean() >= 0.99
    assert np.abs(lse.cpu().numpy()[:, heads] - g["lse"]).max() < 5e-3


@pytest.mark.parametrize("name", cases.I8_GOLDEN)
def test_int8_qk_public_entry_against_the_reference_fixtures(pkg, cuda, name):
    """qk_i8=True (the reference's default mode) through the public entry, against the outputs the
    unmodified reference produced on the same seeded inputs: its quant.py + oracle_a.attention
    composition, and its whole-pipeline INT8 oracle oracle_a.reference where the fixture has it."""
    case = next(c for c in cases.GOLDEN_CASES if c["name"] == name)
    g = np.load(GOLDEN / f"{name}__i8.npz")
    _, _, (out, lse) = _public(pkg, cuda, case, return_lse=True, qk_i8=True)
    _, _, fp8_out = _public(pkg, cuda, case, qk_i8=False)
    assert not torch.equal(out, fp8_out), "the two QK operand types are different operators"
    heads = g["heads"].tolist()
    got = out.float().cpu().numpy()[:, heads]
    for key_o, key_l in (("out_bf16_bits", "lse"), ("oracle_a_out_bf16_bits", "oracle_a_lse")):
        if key_o not in g.files:
            continue
        ref = O.bf16_bits_to_f32(g[key_o])
        rel = H.row_rel(got, ref)
        assert np.median(rel) < 2e-3 and (rel < 9e-3).mean() > 0.97, key_o
        assert np.abs(lse.cpu().numpy()[:, heads] - g[key_l]).max() < 5e-3, key_l


def test_capacity_equals_grow_and_reuse_after_a_larger_request(pkg, cuda):
    small, large = cases.GOLDEN_CASES[1], EXTRA_CASES[0]
    _, args_s, out_fresh = _public(pkg, cuda, small)
    ws = pkg.plan_workspace(cuda, max_kv_len=2048, max_q_len=512, q_heads=small["H"], kv_heads=4)
    before = ws.buffer_pointers()
    out_cap = H.fp8_extend(pkg, *args_s, small["prefix"], sm_scale=small["sm_scale"], workspace=ws)
    assert torch.equal(out_cap, out_fresh)
    # poison every scratch byte with the E4M3 NaN pattern, then rerun: nothing stale may be read
    ws._base.fill_(0x7F)
    ws.view("status").zero_()
    out_again = H.fp8_extend(pkg, *args_s, small["prefix"], sm_scale=small["sm_scale"], workspace=ws)
    assert torch.equal(out_again, out_fresh) and ws.buffer_pointers() == before
    # grow-on-demand workspace reused after a larger request (stale longer data left behind)
    grow = pkg.FP8PrefillWorkspace(cuda)
    inp_l = cases.make_inputs(large)
    ql, kl, vl, il = H.to_dev(inp_l, cuda)
    big1 = H.fp8_extend(pkg, ql, kl, vl, il, large["prefix"], sm_scale=large["sm_scale"], workspace=grow)
    small_on_24 = cases._case("s24", 37, 65, 28, 24, 4, "scattered", "uniform", 4101)
    inp_s = cases.make_inputs(small_on_24)
    a = H.fp8_extend(pkg, *H.to_dev(inp_s, cuda), 28, workspace=grow)
    b = H.fp8_extend(pkg, *H.to_dev(inp_s, cuda), 28)
    assert torch.equal(a, b)
    assert torch.equal(H.fp8_extend(pkg, ql, kl, vl, il, large["prefix"], sm_scale=large["sm_scale"], workspace=grow), big1)
    with pytest.raises(pkg.WorkspaceCapacityError):
        H.fp8_extend(pkg, ql, kl, vl, il, large["prefix"], workspace=pkg.plan_workspace(
            cuda, max_kv_len=1000, max_q_len=512, q_heads=24, kv_heads=4))


def test_foreign_pool_slots_and_index_width_do_not_matter(pkg, cuda):
    """gather == contiguous, NaN in slots the page table does not name, int32 == int64."""
    case = cases.GOLDEN_CASES[3]                                   # scattered fp16 pool, 32:4
    inp = cases.make_inputs(case)
    q, kp, vp, idx = H.to_dev(inp, cuda)
    base = H.fp8_extend(pkg, q, kp, vp, idx, case["prefix"], sm_scale=case["sm_scale"])
    contiguous = H.fp8_extend(pkg, q, kp[idx].contiguous(), vp[idx].contiguous(),
                                    torch.arange(case["N"], device=cuda), case["prefix"], sm_scale=case["sm_scale"])
    assert torch.equal(base, contiguous)
    mask = torch.ones(kp.shape[0], dtype=torch.bool, device=cuda)
    mask[idx] = False
    kp2, vp2 = kp.clone(), vp.clone()
    kp2[mask] = float("nan")
    vp2[mask] = float("nan")
    assert torch.equal(H.fp8_extend(pkg, q, kp2, vp2, idx, case["prefix"], sm_scale=case["sm_scale"]), base)
    assert torch.equal(H.fp8_extend(pkg, q, kp, vp, idx.to(torch.int32), case["prefix"], sm_scale=case["sm_scale"]), base)


def test_gqa_head_map_v_linearity_duplicate_channels_constant_v(pkg, cuda):
    case = cases._case("struct", 96, 300, 204, 24, 4, "scattered", "outlier", 4601)
    inp = cases.make_inputs(case)
    q, kp, vp, idx = H.to_dev(inp, cuda)
    # all six heads of a group carry the same query -> identical outputs inside a group only
    qg = q.clone()
    for grp in range(4):
        qg[:, grp * 6:(grp + 1) * 6] = q[:, grp * 6:grp * 6 + 1]
    out = H.fp8_extend(pkg, qg, kp, vp, idx, case["prefix"])
    for grp in range(4):
        for h in range(grp * 6 + 1, grp * 6 + 6):
            assert torch.equal(out[:, h], out[:, grp * 6])
    assert not torch.equal(out[:, 0], out[:, 6])
    # swapping kv heads 1 and 2 in the pool swaps the outputs of their query groups
    perm = [0, 2, 1, 3]
    out_sw = H.fp8_extend(pkg, qg, kp[:, perm].contiguous(), vp[:, perm].contiguous(), idx, case["prefix"])
    assert torch.equal(out_sw[:, 0:6], out[:, 0:6])
    qsw = qg.clone()
    qsw[:, 6:12], qsw[:, 12:18] = qg[:, 12:18], qg[:, 6:12]
    out_sw2 = H.fp8_extend(pkg, qsw, kp[:, perm].contiguous(), vp[:, perm].contiguous(), idx, case["prefix"])
    assert torch.equal(out_sw2[:, 6:12], out[:, 12:18]) and torch.equal(out_sw2[:, 12:18], out[:, 6:12])
    # O(2V) == 2 O(V): a power-of-two scale moves no byte, only the scales
    base = H.fp8_extend(pkg, q, kp, vp, idx, case["prefix"])
    twice = H.fp8_extend(pkg, q, kp, (vp.float() * 2).to(vp.dtype), idx, case["prefix"])
    assert torch.equal(twice.float(), base.float() * 2)
    # duplicated V channels give identical output channels
    vd = vp.clone()
    vd[:, :, 128:] = vd[:, :, :128]
    dup = H.fp8_extend(pkg, q, kp, vd, idx, case["prefix"])
    assert torch.equal(dup[:, :, 128:], dup[:, :, :128])
    # constant V: centred V is zero, the output is the mean, exactly
    vc = torch.full_like(vp, 0.375)
    const = H.fp8_extend(pkg, q, kp, vc, idx, case["prefix"])
    assert bool((const == 0.375).all())


def test_determinism_and_stream_semantics(pkg, cuda):
    case = EXTRA_CASES[0]
    inp = cases.make_inputs(case)
    q, kp, vp, idx = H.to_dev(inp, cuda)
    ws = pkg.plan_workspace(cuda, max_kv_len=case["N"], max_q_len=case["T"], q_heads=24, kv_heads=4)
    a = H.fp8_extend(pkg, q, kp, vp, idx, case["prefix"], workspace=ws)
    outs = [torch.empty_like(q) for _ in range(3)]
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")             # steady state must not synchronise
    try:
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for o in outs:
                H.fp8_extend(pkg, q, kp, vp, idx, case["prefix"], workspace=ws, out=o)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    side.synchronize()
    for o in outs:
        assert torch.equal(o, a)
    assert ws.status() == 0


def test_cuda_graph_capture_replay_changed_values_and_poisoned_scratch(pkg, cuda):
    """Capacity-reserved workspace + caller-owned outputs under one CUDA graph (the pattern of
    the reference's tests/kernel/test_cuda_graph_capacity.py:269-349)."""
    case = cases._case("graph", 200, 1100, 900, 24, 4, "scattered", "outlier", 4701)
    inp = cases.make_inputs(case)
    q, kp, vp, idx = H.to_dev(inp, cuda)
    ws = pkg.plan_workspace(cuda, max_kv_len=1200, max_q_len=256, q_heads=24, kv_heads=4)
    out = torch.empty_like(q)
    lse = torch.empty((case["T"], 24), dtype=torch.float32, device=cuda)
    eager = H.fp8_extend(pkg, q, kp, vp, idx, case["prefix"], workspace=ws, return_lse=True)
    eager = (eager[0].clone(), eager[1].clone())
    ptrs = ws.buffer_pointers()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        H.fp8_extend(pkg, q, kp, vp, idx, case["prefix"], workspace=ws, out=out, lse_out=lse, return_lse=True)
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph):
        H.fp8_extend(pkg, q, kp, vp, idx, case["prefix"], workspace=ws, out=out, lse_out=lse, return_lse=True)
    out.fill_(float("nan"))
    lse.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager[0]) and torch.equal(lse, eager[1]) and ws.buffer_pointers() == ptrs
    # new values in the same buffers
    q.copy_((q.float() * 0.5 + 0.25).to(q.dtype))
    kp.copy_(kp.flip(0))
    vp.copy_((vp.float() * -1.5).to(vp.dtype))
    graph.replay()
    torch.cuda.synchronize()
    fresh = H.fp8_extend(pkg, q, kp, vp, idx, case["prefix"], return_lse=True)
    assert torch.equal(out, fresh[0]) and torch.equal(lse, fresh[1])
    # scratch poisoned with the E4M3 NaN byte between replays
    for name in ("k8", "v8t", "q8"):
        ws.view(name).fill_(0x7F)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, fresh[0]) and ws.status() == 0


def test_batch_over_streams_equals_one_by_one_and_can_be_captured(pkg, cuda):
    """Independent requests spread over two streams/workspaces give byte-identical results, and
    the fork/join is capturable in one CUDA graph."""
    shapes = [(37, 65, 28), (200, 1100, 900), (64, 320, 256), (130, 700, 500), (5, 5, 0)]
    reqs, single = [], []
    for i, (t, n, p) in enumerate(shapes):
        case = cases._case(f"b{i}", t, n, p, 24, 4, "scattered", "outlier", 5200 + i)
        inp = cases.make_inputs(case)
        q, kp, vp, idx = H.to_dev(inp, cuda)
        reqs.append({"q": q, "k_pool": kp, "v_pool": vp, "idx": idx, "prefix": p,
                     "out": torch.empty_like(q), "lse_out": torch.empty((t, 24), dtype=torch.float32, device=cuda)})
        single.append(H.fp8_extend(pkg, q, kp, vp, idx, p, return_lse=True))
    wss = [pkg.plan_workspace(cuda, max_kv_len=1200, max_q_len=256, q_heads=24, kv_heads=4) for _ in range(2)]
    res = H.fp8_batch(pkg, reqs, workspace=wss, return_lse=True)
    torch.cuda.synchronize()
    for (o, l), (so, sl), r in zip(res, single, reqs):
        assert o is r["out"] and torch.equal(o, so) and torch.equal(l, sl)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        H.fp8_batch(pkg, reqs, workspace=wss, return_lse=True)
    for r in reqs:
        r["out"].fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    for r, (so, sl) in zip(reqs, single):
        assert torch.equal(r["out"], so) and torch.equal(r["lse_out"], sl)
    assert all(w.status() == 0 for w in wss)


# ------------------------------------------------------------------ full-size properties (config 2 shapes)
def test_main_profile_shape_sampled_oracle_and_properties(pkg, cuda):
    """One request of the main 24:4 profile at its deepest (prefix 8192, 2048 new tokens):
    determinism, gather == contiguous, O(2V) = 2 O(V), and the float64 oracle on two heads."""
    T, P, Hq, KVH = 2048, 8192, 24, 4
    N = T + P
    q = cases.outlier_normal((T, Hq, 256), cases.object_seed(2, 0, 0)).to(torch.bfloat16)
    k = cases.outlier_normal((N, KVH, 256), cases.object_seed(2, 0, 1)).to(torch.bfloat16)
    v = cases.outlier_normal((N, KVH, 256), cases.object_seed(2, 0, 2)).to(torch.bfloat16)
    gperm = torch.Generator().manual_seed(cases.object_seed(2, 0, 3))
    pool = 16384
    idx = torch.randperm(pool, generator=gperm)[:N]
    kp = torch.zeros(pool, KVH, 256, dtype=torch.bfloat16)
    vp = torch.zeros(pool, KVH, 256, dtype=torch.bfloat16)
    kp[idx], vp[idx] = k, v
    qd, kd, vd, idd = q.to(cuda), kp.to(cuda), vp.to(cuda), idx.to(cuda)
    ws = pkg.plan_workspace(cuda, max_kv_len=N, max_q_len=T, q_heads=Hq, kv_heads=KVH)
    out, lse = H.fp8_extend(pkg, qd, kd, vd, idd, P, sm_scale=1 / 16, workspace=ws, return_lse=True)
    out, lse = out.clone(), lse.clone()
    assert torch.equal(H.fp8_extend(pkg, qd, kd, vd, idd, P, sm_scale=1 / 16, workspace=ws), out)
    assert torch.equal(H.fp8_extend(pkg, qd, k.to(cuda), v.to(cuda), torch.arange(N, device=cuda), P,
                                          sm_scale=1 / 16, workspace=ws), out)
    twice = H.fp8_extend(pkg, qd, kd, (vd.float() * 2).to(torch.bfloat16), idd, P, sm_scale=1 / 16, workspace=ws)
    assert torch.equal(twice.float(), out.float() * 2)
    H.fp8_extend(pkg, qd, kd, vd, idd, P, sm_scale=1 / 16, workspace=ws)
    torch.cuda.synchronize()
    assert ws.status() == 0
    qp, kv = H.workspace_packs(ws, T, N)
    twin = O.preprocess_kv(k.float().numpy(), v.float().numpy())
    assert np.array_equal(kv.k8, twin.k8) and np.array_equal(kv.v8, twin.v8)
    assert np.array_equal(bits(kv.kscale), bits(twin.kscale)) and np.array_equal(bits(kv.vst), bits(twin.vst))
    heads = [0, 23]
    ref, ref_lse = O.attention(qp, kv, P, T, Hq // KVH, return_lse=True, heads=heads)
    got = out.float().cpu().numpy()[:, heads]
    assert np.abs(lse.cpu().numpy()[:, heads] - ref_lse).max() < 5e-3
    ok = H.output_within_bound(got, ref)
    rel = H.row_rel(got, ref)
    # rows with a flipped P byte are the only ones allowed outside; count them instead of dumping
    inside = ok.reshape(T, len(heads), 256).all(axis=2)
    H.record("attention_vs_oracle", "main_profile_depth_prefix8192_T2048/fp8", rows=int(inside.size),
             rows_outside_output_bound=int((~inside).sum()), rows_over_9e_3=int((rel >= 9e-3).sum()),
             rowrel_median=float(np.median(rel)), rowrel_max=float(rel.max()), max_over_rms=H.max_over_rms(got, ref),
             lse_max_abs=float(np.abs(lse.cpu().numpy()[:, heads] - ref_lse).max()))
    assert inside.mean() >= 0.995                     # observed: every row inside
    assert np.median(rel) < 1.5e-3 and (rel < 9e-3).mean() >= 0.998      # observed: none over, max 4.6e-3


# ------------------------------------------------------------------ properties ported from the reference's tests
def test_oracle_comparison_is_sensitive_to_a_three_percent_scale_error(pkg, cuda):
    """The comparison above must be able to fail: one K tile's scale off by 3 % in the workspace,
    between the transform and the attention launch, has to break the row-relative bound
    (the reference's sensitivity check, tests/kernel/test_oracle_a.py:201-219)."""
    import ctypes

    from attn_kernel_lab_b200 import kernel as K, quant

    case = cases.GOLDEN_CASES[0]
    inp = cases.make_inputs(case)
    q, kp, vp, idx = H.to_dev(inp, cuda)
    ws = pkg.FP8PrefillWorkspace(cuda)
    out, lse, _ = H.run_phases(pkg, ws, q, kp, vp, idx, case["prefix"], case["sm_scale"])
    qp, kv = H.workspace_packs(ws, case["T"], case["N"])
    ref = O.attention(qp, kv, case["prefix"], case["T"], case["H"] // case["KVH"])
    clean = H.row_rel(out.float().cpu().numpy(), ref)
    assert (clean < 9e-3).mean() >= 0.995
    lib = K.load()
    call = quant.make_call(ws, q=q, k_pool=kp, v_pool=vp, idx=idx, out=out, lse_out=lse, q_len=case["T"],
                           kv_len=case["N"], prefix=case["prefix"], q_heads=case["H"], kv_heads=case["KVH"],
                           sm_scale=case["sm_scale"])
    ws.view("kscale")[:, 1] *= 1.03                 # every kv head, second 64-key tile
    K.check(lib.akl_attention(ctypes.byref(call), torch.cuda.current_stream().cuda_stream), "akl_attention")
    torch.cuda.synchronize()
    broken = H.row_rel(out.float().cpu().numpy(), ref)
    assert np.median(broken) > 3 * np.median(clean) and (broken >= 9e-3).mean() > 0.2, \
        "a 3 % scale error went unnoticed: the comparison has no teeth"


def test_future_keys_are_invisible(pkg, cuda):
    """Changing K at the last position (no K centring, so no request-wide statistic of K moves;
    V untouched) may change only rows that can see that position's 64-key tile: the tile's scale
    and bytes change, nothing before it does (after tests/kernel/test_divergence_hunting.py:434-460)."""
    T, N, prefix, Hq, KVH = 200, 1000, 800, 24, 4
    q = cases.outlier_normal((T, Hq, 256), 4501).to(torch.bfloat16).to(cuda)
    k = cases.outlier_normal((N, KVH, 256), 4502).to(torch.bfloat16).to(cuda)
    v = cases.outlier_normal((N, KVH, 256), 4503).to(torch.bfloat16).to(cuda)
    idx = torch.arange(N, device=cuda)
    base, base_lse = H.fp8_extend(pkg, q, k, v, idx, prefix, sm_scale=1 / 16, center_k=False, return_lse=True)
    k2 = k.clone()
    k2[N - 1] = (k2[N - 1].float() * 3 + 1).to(torch.bfloat16)
    other, other_lse = H.fp8_extend(pkg, q, k2, v, idx, prefix, sm_scale=1 / 16, center_k=False, return_lse=True)
    last_tile_start = (N - 1) // 64 * 64                      # rows whose reach ends before this tile are untouched
    untouched = [r for r in range(T) if prefix + r < last_tile_start]
    assert len(untouched) > 100
    assert torch.equal(base[untouched].view(torch.int16), other[untouched].view(torch.int16))
    assert torch.equal(base_lse[untouched].view(torch.int32), other_lse[untouched].view(torch.int32))
    assert not torch.equal(base[T - 1], other[T - 1])         # the last row sees the changed key


@pytest.mark.parametrize("sm_scale", [1 / 64, 1 / 16, 0.11, 1.0])
def test_softmax_scale_is_folded_exactly_once(pkg, cuda, sm_scale):
    """The scale enters only through the Q scales (quant.py:479): the operator at sm_scale must match
    the float64 oracle at the same sm_scale (after tests/kernel/test_divergence_hunting.py:979-995)."""
    case = dict(cases.GOLDEN_CASES[2])                        # 100 rows over 200 keys, 16:4
    inp = cases.make_inputs(case)
    q, kp, vp, idx = H.to_dev(inp, cuda)
    out, lse = H.fp8_extend(pkg, q, kp, vp, idx, case["prefix"], sm_scale=sm_scale, return_lse=True)
    qf, kf, vf = H.gathered(inp)
    ref, ref_lse = O.reference(qf, kf, vf, case["prefix"], sm_scale=sm_scale, return_lse=True)
    rel = H.row_rel(out.float().cpu().numpy(), ref)
    H.record("sm_scale_sweep", f"ragged_100_200/{sm_scale:.4g}", rowrel_median=float(np.median(rel)),
             rowrel_max=float(rel.max()), rows_over_9e_3=int((rel >= 9e-3).sum()), rows=int(rel.size))
    assert np.median(rel) < 2e-3 and (rel < 9e-3).mean() >= 0.97
    assert np.abs(lse.cpu().numpy() - ref_lse).max() < 5e-3


# ------------------------------------------------------------------ KV-axis split and merge
def test_merge_kernel_against_the_float64_merge(pkg, cuda):
    from attn_kernel_lab_b200 import dist as D

    g = torch.Generator().manual_seed(4801)
    rows, parts = 3000, 5
    os_ = [torch.randn(rows, 256, generator=g).to(torch.bfloat16) for _ in range(parts)]
    ls = [torch.randn(rows, generator=g) * 6 for _ in range(parts)]
    ls[1][::7] = float("-inf")
    ls[3][:100] = float("-inf")
    for l in ls:
        l[5] = float("-inf")                          # a row no split saw
    out, lse = D.merge_states([o.to(cuda) for o in os_], [l.to(cuda) for l in ls])
    want_o, want_l = O.merge_splits([o.float().numpy() for o in os_], [l.numpy() for l in ls])
    got = out.float().cpu().numpy()
    keep = np.ones(rows, bool)
    keep[5] = False
    assert np.abs(got[keep] - want_o[keep]).max() <= 2 * H.bf16_ulp(want_o[keep]).max()
    assert (np.abs(got[keep] - want_o[keep]) <= 1.01 * H.bf16_ulp(want_o[keep])).all()
    assert np.allclose(lse.cpu().numpy()[keep], want_l[keep], atol=2e-6)
    assert np.isneginf(lse.cpu().numpy()[5]) and torch.equal(out[5].cpu(), os_[0][5])


def test_kv_axis_split_emulated_on_one_gpu(pkg, cuda):
    """The multi-GPU KV split run as consecutive split calls on one device (ranks that wait on
    one another never share a GPU): request-wide statistics through the shared tile-sum arrays,
    per-split attention with global causal positions, merge kernel.  Oracle: the per-split
    operator with request-wide statistics + float64 merge."""
    from attn_kernel_lab_b200 import dist as D

    case = cases._case("split_gpu", 192, 3400, 3208, 32, 4, "scattered", "outlier", 4901)
    inp = cases.make_inputs(case)
    q, kp, vp, idx = H.to_dev(inp, cuda)
    n_total, T, prefix = case["N"], case["T"], case["prefix"]
    merged, mlse, wss, ranges, outs, lses = H.emulated_kv_split(pkg, q, kp, vp, idx, prefix, case["sm_scale"], 4)
    assert ranges[-1][1] == n_total and ranges[2][1] - ranges[2][0] > 0

    qf, kf, vf = H.gathered(inp)
    whole = O.preprocess_kv(kf, vf)
    assert np.array_equal(bits(wss[0].view("kmean").cpu().numpy()), bits(whole.kmean))
    assert np.array_equal(bits(wss[3].view("vmean").cpu().numpy()), bits(whole.vmean))
    for ws, (lo, hi) in zip(wss, ranges):             # every split holds the request-wide bytes of its range
        assert np.array_equal(ws.k8_logical(hi - lo).cpu().numpy()[:, :hi - lo], whole.k8[:, lo:hi])
        assert np.array_equal(ws.v8_logical(hi - lo).cpu().numpy()[:, :hi - lo], whole.v8[:, lo:hi])
    qp = O.preprocess_q(qf, case["sm_scale"])
    ref_parts = [O.attention(qp, whole, prefix, T, 8, return_lse=True, kv_lo=lo, kv_hi=hi) for lo, hi in ranges]
    for (ro, rl), o, l in zip(ref_parts, outs, lses):
        gl = l.cpu().numpy()
        assert np.array_equal(np.isneginf(gl), np.isneginf(rl))
        fin = np.isfinite(rl)
        assert np.abs(gl[fin] - rl[fin]).max() < 5e-3
        rel = H.row_rel(o.float().cpu().numpy(), ro).reshape(T, 32)
        assert np.median(rel[fin]) < 2e-3 and (rel[fin] < 9e-3).mean() > 0.95
    want_o, want_l = O.merge_splits([p[0] for p in ref_parts], [p[1] for p in ref_parts])
    rel = H.row_rel(merged.float().cpu().numpy(), want_o)
    assert np.median(rel) < 2e-3 and (rel < 9e-3).mean() > 0.95
    assert np.abs(mlse.cpu().numpy() - want_l).max() < 5e-3
    # distance to the unsplit operator, reported by the split oracle test: same LSE, P-noise apart
    single = H.fp8_extend(pkg, q, kp, vp, idx, prefix, sm_scale=case["sm_scale"], return_lse=True)
    assert np.abs(single[1].cpu().numpy() - mlse.cpu().numpy()).max() < 5e-3
