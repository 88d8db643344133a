"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations, shared by the benchmark and the tests.

Value recipes follow the reference's own generators: N(0,1) with 2 % of channels scaled x16 for the
throughput profiles (bench/candidate_bench.py:218-263 of the reference), N(0, 0.5) with per-token
norm jitter for the GQA sweep, and a planted rank-8 attention sink for the long single request.
Length recipes follow the five configurations: main 24:4 profile, GQA sweep, long single request,
serving batch.  All draws use a CPU torch.Generator so the vectors do not depend on the device.
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
