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

HEAD_DIM = 256
BASE_SEED = 20260829


def object_seed(config: int, request: int = 0, obj: int = 0, layer: int = 0) -> int:
    """base + 1000*config + 10*request + {0:q,1:k,2:v,3:perm,4:lens} + 100000*layer."""
    return BASE_SEED + 1000 * config + 10 * request + obj + 100000 * layer


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(int(seed))


def outlier_normal(shape, seed: int, frac: float = 0.02, gain: float = 16.0, sigma: float = 1.0):
    """N(0, sigma) with a seeded `frac` of the 256 channels (at least one) scaled by `gain`."""
    g = _gen(seed)
    x = torch.randn(shape, generator=g) * sigma
    mask = torch.rand(HEAD_DIM, generator=g) < frac
    if not bool(mask.any()):
        mask[int(torch.randint(0, HEAD_DIM, (1,), generator=g))] = True
    x[..., mask] *= gain
    return x


def jitter_normal(shape, seed: int, sigma: float = 0.5):
    """N(0, sigma) with every token row scaled by u ~ U(0.5, 2)."""
    g = _gen(seed)
    x = torch.randn(shape, generator=g) * sigma
    u = torch.rand(shape[0], generator=g) * 1.5 + 0.5
    return x * u.view(-1, *([1] * (len(shape) - 1)))


def uniform_pm1(shape, g: torch.Generator):
    return torch.rand(shape, generator=g) * 2 - 1


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


# --------------------------------------------------------------------------
# the benchmark configurations (seeded stand-ins for the reference's synthetic schedule)
# --------------------------------------------------------------------------

def c2_lengths(num_requests: int = 8, seed: int | None = None):
    """Main 24:4 profile: prefix_i ~ U{1024..8192}, 2048 extend tokens each."""
    g = _gen(object_seed(2, 0, 4) if seed is None else seed)
    prefixes = torch.randint(1024, 8193, (num_requests,), generator=g).tolist()
    return [(int(p), 2048) for p in prefixes]


def c3_lengths(num_requests: int = 16, seed: int | None = None):
    """GQA sweep: T_i log-uniform in [1, 4096], prefix_i ~ U{0..16384}."""
    g = _gen(object_seed(3, 0, 4) if seed is None else seed)
    u = torch.rand(num_requests, generator=g)
    ts = torch.exp(u * math.log(4096.0)).round().clamp(1, 4096).to(torch.int64).tolist()
    prefixes = torch.randint(0, 16385, (num_requests,), generator=g).tolist()
    return [(int(p), int(t)) for p, t in zip(prefixes, ts)]


def c5_lengths(num_requests: int = 256, seed: int | None = None):
    """Serving batch: T_i ~ Geometric(mean 128) capped at 512, prefix_i ~ U{0..32768}."""
    g = _gen(object_seed(5, 0, 4) if seed is None else seed)
    u = torch.rand(num_requests, generator=g).clamp_min(1e-12)
    ts = (torch.log(u) / math.log(1.0 - 1.0 / 128.0)).floor().to(torch.int64) + 1
    ts = ts.clamp(1, 512).tolist()
    prefixes = torch.randint(0, 32769, (num_requests,), generator=g).tolist()
    return [(int(p), int(t)) for p, t in zip(prefixes, ts)]


def run_page_table(pool_rows: int, n: int, run: int, seed: int) -> torch.Tensor:
    """Pool cut into `run`-slot contiguous runs, runs randomly permuted; positions walk
    the runs in that order (config 4: 64-slot runs)."""
    nruns = pool_rows // run
    order = torch.randperm(nruns, generator=_gen(seed))
    table = (order[:, None] * run + torch.arange(run)[None, :]).reshape(-1)
    return table[:n].to(torch.int64)


def sink_qk(T: int, N: int, H: int, KVH: int, seed: int):
    """Config 4 values: Q/K ~ N(0,1) plus a planted rank-8 sink on the first 4 keys."""
    g = _gen(seed)
    q = torch.randn((T, H, HEAD_DIM), generator=g)
    k = torch.randn((N, KVH, HEAD_DIM), generator=g)
    basis, _ = torch.linalg.qr(torch.randn((HEAD_DIM, 8), generator=g))
    w = torch.randn((4, 8), generator=g)
    k[:4] += 4.0 * (w @ basis.T)[:, None, :]
    wbar = w.mean(dim=0)
    q += 2.0 * (basis @ (wbar / wbar.norm()))[None, None, :]
    return q.to(torch.bfloat16), k.to(torch.bfloat16)


def attention_flops(H: int, T: int, prefix: int, D: int = HEAD_DIM) -> float:
    """4*Hq*D*T*(prefix + (T+1)/2): logically attended pairs
    (reference bench/candidate_bench.py:210-212, tools/gen_workload.py:69-73)."""
    return 4.0 * H * D * T * (prefix + (T + 1) / 2.0)
