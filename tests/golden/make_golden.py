"""Regenerate the golden fixtures in this directory by RUNNING THE REFERENCE ITSELF.

Run in a container that has the reference checkout (it is imported, never copied):

    python tests/golden/make_golden.py --reference /path/to/attn-kernel-lab

For every case the script draws seeded inputs on the CPU, runs the reference's own
FP8-QK composition -- quant.gather_quantize_kv(qk_i8=False) + quant.quantize_q(qk_i8=False)
wrapped as oracle_a.QPack / KVPack and fed to oracle_a.attention, the pattern of the
reference's tests/kernel/test_ops_gpu.py:48-68 -- and stores what came out:

    <case>.npz   inputs' sha256, quantised artifacts (bytes or sha256), scales, means,
                 fold arrays, and the BF16 output + base-2 LSE for a subset of heads.

For the cases named in cases.I8_GOLDEN the same is done once more with qk_i8=True (the
reference's default INT8-QK mode) into <case>__i8.npz, together with the output of the
reference's own INT8 oracle oracle_a.reference on the same inputs.

It also extracts, as plain data, the k8 / vt8 / q8 sha256 digests of the FP8-QK,
fp8-PV single-shot cases of the reference's tests/kernel/golden_bitexact.json (and, under
"cases_i8", of its INT8-QK cases) into bitexact_digests.json (digests only; the case recipe is restated in tests/cases.py).

The fixtures travel with the repository; the reference checkout does not.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
import cases as case_mod  # noqa: E402  (tests/cases.py: seeded input recipes)


def sha(t) -> str:
    if isinstance(t, torch.Tensor):
        t = t.detach().cpu().contiguous()
        if t.dtype != torch.uint8:
            t = t.view(torch.uint8)
        return hashlib.sha256(t.numpy().tobytes()).hexdigest()
    return hashlib.sha256(np.ascontiguousarray(t).tobytes()).hexdigest()


def run_reference(ref_src: pathlib.Path, case: dict, qk_i8: bool = False) -> dict:
    sys.path.insert(0, str(ref_src))
    from attn_kernel_lab import oracle_a, quant  # the reference, unmodified

    inp = case_mod.make_inputs(case)
    q, k_pool, v_pool, idx = inp["q"], inp["k_pool"], inp["v_pool"], inp["idx"]
    T, H, D = q.shape
    KVH = k_pool.shape[1]
    N = idx.numel()
    sm_scale = case["sm_scale"]
    ws = quant.FP8PrefillWorkspace(torch.device("cpu"))
    kvd = quant.gather_quantize_kv(
        ws, k_pool, v_pool, idx.long(), need_vt8=True, need_vb16=False,
        center_k=case["center_k"], qk_i8=qk_i8, rotate=case["rotate"],
    )
    q8, qscale, mpad = quant.quantize_q(ws, q, sm_scale, qk_i8=qk_i8, rotate=case["rotate"])
    npad = kvd["ntmax"] * quant.BLK
    nt = kvd["ntmax"]
    ksum = ws.get("ksum", (KVH, D), torch.float32).clone()
    kmean = ksum / max(N, 1) if case["center_k"] else torch.zeros_like(ksum)
    vst = ws.get("vscale_t", (KVH, nt), torch.float32).clone()

    # logical (position-order) V bytes: undo the SIGMA permutation + transpose
    sigma = torch.tensor(quant.SIGMA64, dtype=torch.long)
    inv = torch.empty_like(sigma)
    inv[sigma] = torch.arange(quant.BLK)
    vt8 = kvd["vt8"].view(KVH, nt, D, quant.BLK)
    v8_logical = vt8.permute(0, 1, 3, 2).index_select(2, inv).reshape(KVH, npad, D).contiguous()

    qk_view = torch.int8 if qk_i8 else torch.float8_e4m3fn
    qp = oracle_a.QPack(q8=q8.view(qk_view), qscale=qscale, mpad=mpad)
    kvp = oracle_a.KVPack(
        k8=kvd["k8"].view(qk_view), kscale=kvd["kscale"], kmean=kmean,
        vt8=vt8.view(torch.float8_e4m3fn), vst_scaled=vst, vscale=kvd["vscale"],
        vlog2r=kvd["vlog2r"], vinvr=kvd["vinvr"], vmean=kvd["vmean"], n=N,
    )
    out, lse = oracle_a.attention(qp, kvp, case["prefix"], T, group=H // KVH, return_lse=True)

    heads = case_mod.golden_heads(H, KVH)
    rec = {
        "in_sha_q": sha(q), "in_sha_k_pool": sha(k_pool), "in_sha_v_pool": sha(v_pool),
        "in_sha_idx": sha(idx.long()),
        "qscale": qscale.numpy().copy(), "kscale": kvd["kscale"].numpy().copy(),
        "kmean": kmean.numpy().copy(), "vmean": kvd["vmean"].numpy().copy(),
        "vst": vst.numpy().copy(), "vscale": kvd["vscale"].numpy().copy(),
        "vlog2r": kvd["vlog2r"].numpy().copy(), "vinvr": kvd["vinvr"].numpy().copy(),
        "sha_q8": sha(q8), "sha_k8": sha(kvd["k8"]), "sha_v8": sha(v8_logical),
        "heads": np.asarray(heads, np.int32),
        "out_bf16_bits": out[:, heads].contiguous().view(torch.int16).numpy().view(np.uint16).copy(),
        "lse": lse[:, heads].numpy().copy(),
    }
    if qk_i8 and case["rotate"] and case["center_k"]:
        # the reference's own INT8 oracle, whole pipeline, on the gathered rows
        rows = idx.long()
        own, own_lse = oracle_a.reference(q, k_pool[rows], v_pool[rows], case["prefix"], sm_scale=sm_scale,
                                          return_lse=True)
        rec["oracle_a_out_bf16_bits"] = own[:, heads].contiguous().view(torch.int16).numpy().view(np.uint16).copy()
        rec["oracle_a_lse"] = own_lse[:, heads].numpy().copy()
    if case.get("store_bytes", False):
        rec["q8"] = q8.numpy().copy()
        rec["k8"] = kvd["k8"].numpy().copy()
        rec["v8"] = v8_logical.numpy().copy()
    return rec


def extract_bitexact(ref_root: pathlib.Path) -> dict:
    j = json.loads((ref_root / "tests" / "kernel" / "golden_bitexact.json").read_text())
    keep, keep_i8 = {}, {}
    for cid, c in j["cases"].items():
        m = c["meta"]
        if m["pv"] != "fp8" or m["chunks"] is not None:
            continue
        (keep_i8 if m["qk_i8"] else keep)[cid] = {
            "meta": {k: m[k] for k in ("shape", "T", "N", "prefix", "H", "KVH", "pool",
                                       "seed", "rotate", "center_k")},
            "artifacts": {k: c["artifacts"][k] for k in ("q8", "k8", "vt8")},
        }
    return {"source": "tests/kernel/golden_bitexact.json (reference), FP8-QK fp8-PV single-shot cases",
            "env": j["env"], "cases": keep, "cases_i8": keep_i8}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout (attn-kernel-lab)")
    args = ap.parse_args()
    ref_root = pathlib.Path(args.reference)
    torch.set_num_threads(max(1, torch.get_num_threads()))
    for case in case_mod.GOLDEN_CASES:
        rec = run_reference(ref_root / "src", case)
        path = HERE / f"{case['name']}.npz"
        np.savez_compressed(path, **rec)
        print(f"{case['name']}: wrote {path.name} ({path.stat().st_size / 1024:.0f} KiB)")
        if case["name"] in case_mod.I8_GOLDEN:
            rec = run_reference(ref_root / "src", case, qk_i8=True)
            path = HERE / f"{case['name']}__i8.npz"
            np.savez_compressed(path, **rec)
            print(f"{case['name']} (INT8 QK): wrote {path.name} ({path.stat().st_size / 1024:.0f} KiB)")
    (HERE / "bitexact_digests.json").write_text(json.dumps(extract_bitexact(ref_root), indent=1))
    print("wrote bitexact_digests.json")


if __name__ == "__main__":
    main()
