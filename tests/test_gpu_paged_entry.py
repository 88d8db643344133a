"""FlashInfer-shaped entry on the GPU: the accuracy matrix against unquantised float64 attention at
the reference's thresholds, and the equalities that are not tolerance questions -- page-map
equivalence, pages no index names, workspace reuse, `out=` identity -- at zero tolerance
(upstream/pr-draft/tests/attention/test_fp8_paged_prefill_sm120.py:185-393, 468-488)."""
import numpy as np
import pytest
import torch

import akl_oracle as O
import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture()
def entry(pkg):
    from attn_kernel_lab_b200 import paged
    return paged.fp8_paged_prefill


def _uniform(shape, g, dev, dtype=torch.bfloat16):
    return torch.empty(shape, dtype=torch.float32).uniform_(-1.0, 1.0, generator=g).to(dtype).to(dev)


def make_request(qo, kv, dev, hq=24, hkv=4, page_map="contiguous", seed=0, filler_seed=None):
    """Position i lives in page i (contiguous), in a random page (shuffled), or in page 2i+1 of a
    cache twice the size whose even pages no index names (fragmented).  The logical tensors are
    drawn before the page map, so the same seed gives the same request under every map."""
    g = torch.Generator().manual_seed(seed)
    q = _uniform((qo, hq, 256), g, dev)
    k_log = _uniform((kv, hkv, 256), g, dev)
    v_log = _uniform((kv, hkv, 256), g, dev)
    if page_map == "contiguous":
        rows, pages = torch.arange(kv), kv
    elif page_map == "shuffled":
        rows, pages = torch.randperm(kv, generator=g), kv
    else:
        rows, pages = torch.arange(kv) * 2 + 1, 2 * kv
    fg = g if filler_seed is None else torch.Generator().manual_seed(filler_seed)
    kc = _uniform((pages, 1, hkv, 256), fg, dev)
    vc = _uniform((pages, 1, hkv, 256), fg, dev)
    rows = rows.to(dev)
    kc[rows, 0] = k_log
    vc[rows, 0] = v_log
    return q, kc, vc, rows.to(torch.int64), k_log, v_log


def fp64(q, k_log, v_log):
    return O.plain_attention(q.float().cpu().numpy(), k_log.float().cpu().numpy(),
                             v_log.float().cpu().numpy(), k_log.shape[0] - q.shape[0], 1.0 / 16.0)


def cos_sim(a, b):
    a, b = a.astype(np.float64).ravel(), b.ravel()
    return float(a @ b / max(np.linalg.norm(a) * np.linalg.norm(b), 1e-12))


@pytest.mark.parametrize("qo, kv, cos_min, rel_mean, rel_max", [
    (64, 64, 0.995, 0.06, 0.20),          # no prefix: the shallow corner
    (64, 1024, 0.998, 0.05, 0.15),        # prefix-cache geometry
    (128, 4096, 0.998, 0.05, 0.15),
    (100, 999, 0.998, 0.05, 0.15),        # neither length a multiple of 64 or 128
    (193, 4993, 0.998, 0.05, 0.15),
    (37, 2011, 0.998, 0.05, 0.16),
    (1, 977, 0.995, 0.06, 0.20),          # single-row extend
])
def test_accuracy_against_unquantised_float64(entry, cuda, qo, kv, cos_min, rel_mean, rel_max):
    q, kc, vc, idx, k_log, v_log = make_request(qo, kv, cuda, seed=qo + kv)
    given = torch.empty_like(q) if (qo + kv) % 2 else None
    out = entry(q, kc, vc, idx, out=given)
    torch.cuda.synchronize()
    if given is not None:
        assert out is given
    assert out.dtype == torch.bfloat16 and out.shape == (qo, 24, 256) and torch.isfinite(out).all()
    want = fp64(q, k_log, v_log)
    got = out.float().cpu().numpy()
    rel = H.row_rel(got, want)
    assert cos_sim(got, want) >= cos_min
    assert rel.mean() <= rel_mean and rel.max() <= rel_max, (rel.mean(), rel.max())


@pytest.mark.parametrize("hq, hkv", [(16, 4), (24, 4), (32, 4)])
def test_gqa_ratios_and_group_wiring(entry, cuda, hq, hkv):
    q, kc, vc, idx, k_log, v_log = make_request(96, 1500, cuda, hq=hq, hkv=hkv, seed=hq)
    out = entry(q, kc, vc, idx)
    want = fp64(q, k_log, v_log)
    got = out.float().cpu().numpy()
    assert cos_sim(got, want) >= 0.998 and H.row_rel(got, want).mean() <= 0.05
    # perturbing KV head 1 must change exactly the q heads of group 1
    group = hq // hkv
    kc2 = kc.clone()
    kc2[idx, 0, 1] = -kc2[idx, 0, 1]
    out2 = entry(q, kc2, vc, idx)
    torch.cuda.synchronize()
    assert torch.equal(out2[:, :group], out[:, :group])
    assert torch.equal(out2[:, 2 * group:], out[:, 2 * group:])
    assert not torch.equal(out2[:, group:2 * group], out[:, group:2 * group])


@pytest.mark.parametrize("page_map", ["shuffled", "fragmented"])
def test_page_map_equivalence_is_exact(entry, cuda, page_map):
    base = make_request(150, 3000, cuda, page_map="contiguous", seed=11)
    other = make_request(150, 3000, cuda, page_map=page_map, seed=11)
    assert torch.equal(base[4], other[4]) and torch.equal(base[5], other[5])
    a = entry(*base[:4])
    b = entry(*other[:4])
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_pages_no_index_names_are_never_read(entry, cuda):
    clean = make_request(70, 1100, cuda, page_map="fragmented", seed=3, filler_seed=100)
    dirty = make_request(70, 1100, cuda, page_map="fragmented", seed=3, filler_seed=200)
    dirty[1][0::2] = 3.0e38            # huge but finite: one read of it would poison the statistics
    dirty[2][0::2] = -3.0e38
    a = entry(*clean[:4])
    b = entry(*dirty[:4])
    torch.cuda.synchronize()
    assert torch.isfinite(b).all() and torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_workspace_reuse_long_after_short_and_short_after_long(pkg, entry, cuda):
    ws = pkg.FP8PrefillWorkspace(cuda)
    short = make_request(40, 333, cuda, seed=21)
    long = make_request(200, 5000, cuda, seed=22)
    for first, second in ((short, long), (long, short)):
        entry(*first[:4], workspace_buffer=ws)
        reused = entry(*second[:4], workspace_buffer=ws)
        fresh = entry(*second[:4])
        torch.cuda.synchronize()
        assert torch.isfinite(reused).all() and torch.equal(reused.view(torch.int16), fresh.view(torch.int16))


def test_out_identity_and_lse_shape(entry, cuda):
    q, kc, vc, idx, _, _ = make_request(48, 800, cuda, seed=5)
    given = torch.full_like(q, float("nan"))
    returned, lse = entry(q, kc, vc, idx, out=given, return_lse=True)
    allocated = entry(q, kc, vc, idx)
    torch.cuda.synchronize()
    assert returned is given and torch.equal(returned.view(torch.int16), allocated.view(torch.int16))
    assert lse.shape == (48, 24) and lse.dtype == torch.float32 and torch.isfinite(lse).all()
    assert (lse > -1000).all() and (lse < 1000).all()
    with pytest.raises(ValueError):
        entry(q, kc, vc, idx, out=q)              # the destination may not alias the queries
