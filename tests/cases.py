"""Seeded synthetic inputs shared by the fixture generator, the tests and the benchmark.

Value recipes follow the reference's own generators: uniform [-1, 1) BF16 for the
bit-exact matrix (tests/kernel/test_golden_bitexact.py:478-503 of the reference),
N(0,1) with 2 % of channels scaled x16 for the throughput profiles
(bench/candidate_bench.py:218-263), N(0, 0.5) with per-token norm jitter for the GQA
sweep, and a planted rank-8 attention sink for the long single request.  All draws
use a CPU torch.Generator so the vectors do not depend on the device.
"""
from __future__ import annotations

import math

import torch

from attn_kernel_lab_b200.synthetic import (  # noqa: F401  (shared with the benchmark)
    BASE_SEED, HEAD_DIM, _gen, attention_flops, c2_lengths, c3_lengths, c5_lengths, jitter_normal,
    object_seed, outlier_normal, run_page_table, sink_qk, uniform_pm1)


def golden_heads(H: int, KVH: int):
    """Query heads whose outputs a fixture stores: first, first of the second group, last."""
    g = H // KVH
    return sorted({0, min(g, H - 1), H - 1})


# --------------------------------------------------------------------------
# small cases run through the real reference by tests/golden/make_golden.py
# --------------------------------------------------------------------------

def _case(name, T, N, prefix, H, KVH, pool, dist, seed, *, rotate=True, center_k=True,
          kv_dtype="bfloat16", sm_scale=None, store_bytes=False, pool_rows=None):
    return dict(name=name, T=T, N=N, prefix=prefix, H=H, KVH=KVH, pool=pool, dist=dist,
                seed=seed, rotate=rotate, center_k=center_k, kv_dtype=kv_dtype,
                sm_scale=(1.0 / math.sqrt(HEAD_DIM)) if sm_scale is None else sm_scale,
                store_bytes=store_bytes, pool_rows=pool_rows)


GOLDEN_CASES = [
    # benchmark configuration 1 (the CPU-runnable case): 256 cached + 64 new, 24:4, 4096-slot pool, seeded permutation
    _case("c1_cpu_oracle", 64, 320, 256, 24, 4, "permuted", "outlier", object_seed(1),
          pool_rows=4096, sm_scale=1.0 / 16.0),
    # the reference's oracle-agreement shapes (tests/kernel/test_oracle_a.py:71-109)
    _case("ragged_37_65", 37, 65, 28, 16, 4, "scattered", "uniform", 4101, store_bytes=True),
    _case("ragged_100_200", 100, 200, 100, 16, 4, "contiguous", "outlier", 4102),
    _case("tiles_128_448", 128, 448, 320, 32, 4, "scattered", "jitter", 4103, kv_dtype="float16"),
    _case("subtile_5_5", 5, 5, 0, 16, 4, "contiguous", "uniform", 4104, store_bytes=True),
    # preprocessing variants
    _case("norot_64_128", 64, 128, 64, 16, 4, "contiguous", "outlier", 4105, rotate=False),
    _case("nocen_64_130", 64, 130, 66, 16, 4, "scattered", "outlier", 4106, center_k=False),
]

#: cases that also have a fixture for the reference's INT8-QK mode (<name>__i8.npz)
I8_GOLDEN = ("c1_cpu_oracle", "ragged_37_65", "tiles_128_448", "norot_64_128", "nocen_64_130")


def make_inputs(case: dict) -> dict:
    """q [T,H,D] bf16, k_pool/v_pool [pool,KVH,D] bf16|fp16, idx [N] int64 (CPU tensors)."""
    T, N, H, KVH = case["T"], case["N"], case["H"], case["KVH"]
    seed = case["seed"]
    kvdt = torch.float16 if case["kv_dtype"] == "float16" else torch.bfloat16
    if case["dist"] == "uniform":
        g = _gen(seed)
        q = uniform_pm1((T, H, HEAD_DIM), g)
        k = uniform_pm1((N, KVH, HEAD_DIM), g)
        v = uniform_pm1((N, KVH, HEAD_DIM), g)
    elif case["dist"] == "outlier":
        q = outlier_normal((T, H, HEAD_DIM), seed)
        k = outlier_normal((N, KVH, HEAD_DIM), seed + 1)
        v = outlier_normal((N, KVH, HEAD_DIM), seed + 2)
    elif case["dist"] == "jitter":
        q = jitter_normal((T, H, HEAD_DIM), seed)
        k = jitter_normal((N, KVH, HEAD_DIM), seed + 1)
        v = jitter_normal((N, KVH, HEAD_DIM), seed + 2)
    else:
        raise ValueError(case["dist"])
    q = q.to(torch.bfloat16)
    k = k.to(kvdt)
    v = v.to(kvdt)
    if case["pool"] == "contiguous":
        k_pool, v_pool, idx = k, v, torch.arange(N, dtype=torch.int64)
    else:
        g = _gen(seed + 3)
        pool_rows = case["pool_rows"] or (int(N * 1.7) + 97)
        idx = torch.randperm(pool_rows, generator=g)[:N].to(torch.int64)
        # slots that belong to other requests hold unrelated finite data
        k_pool = uniform_pm1((pool_rows, KVH, HEAD_DIM), g).to(kvdt)
        v_pool = uniform_pm1((pool_rows, KVH, HEAD_DIM), g).to(kvdt)
        k_pool[idx] = k
        v_pool[idx] = v
    return dict(q=q.contiguous(), k_pool=k_pool.contiguous(), v_pool=v_pool.contiguous(), idx=idx)


# --------------------------------------------------------------------------
# the reference's bit-exact matrix recipe (inputs for bitexact_digests.json)
# --------------------------------------------------------------------------

def bitexact_inputs(meta: dict) -> dict:
    """Inputs of one single-shot case of the reference's golden matrix:
    q, k, v drawn in that order from one seeded CPU generator as uniform [-1,1) -> BF16;
    'scattered' places the rows at randperm slots of a pool of int(1.7*N)+97 rows whose
    other rows are uniform noise, drawn from a generator seeded with seed+1."""
    T, N, H, KVH, seed = meta["T"], meta["N"], meta["H"], meta["KVH"], meta["seed"]
    g = _gen(seed)
    q = uniform_pm1((T, H, HEAD_DIM), g).to(torch.bfloat16)
    k = uniform_pm1((N, KVH, HEAD_DIM), g).to(torch.bfloat16)
    v = uniform_pm1((N, KVH, HEAD_DIM), g).to(torch.bfloat16)
    if meta["pool"] == "scattered":
        g2 = _gen(seed + 1)
        pool_n = int(N * 1.7) + 97
        slots = torch.randperm(pool_n, generator=g2)[:N]
        kp = uniform_pm1((pool_n, KVH, HEAD_DIM), g2).to(torch.bfloat16)
        vp = uniform_pm1((pool_n, KVH, HEAD_DIM), g2).to(torch.bfloat16)
        kp[slots] = k
        vp[slots] = v
        return dict(q=q, k_pool=kp, v_pool=vp, idx=slots.to(torch.int64))
    return dict(q=q, k_pool=k, v_pool=v, idx=torch.arange(N, dtype=torch.int64))


