"""FlashInfer-shaped entry, host side: what is refused and with which message, before any device
work (upstream/pr-draft/tests/attention/test_fp8_paged_prefill_sm120.py:401-466)."""
import pytest
import torch


@pytest.fixture()
def paged(pkg):
    from attn_kernel_lab_b200 import paged
    return paged


def _req(qo=8, kv=32, hq=24, hkv=4, d=256, page=1, dtype=torch.bfloat16):
    q = torch.zeros(qo, hq, d, dtype=torch.bfloat16)
    kc = torch.zeros(kv, page, hkv, d, dtype=dtype)
    return q, kc, kc.clone(), torch.arange(kv)


@pytest.mark.parametrize("head_dim", [64, 128, 512])
def test_rejects_head_dim(pkg, paged, head_dim):
    q, kc, vc, idx = _req(d=head_dim)
    with pytest.raises(pkg.CapabilityError) as e:
        paged.fp8_paged_prefill(q, kc, vc, idx)
    assert e.value.field == "head_dim"


def test_rejects_page_size_before_reshaping(pkg, paged):
    q, kc, vc, idx = _req(page=16)
    with pytest.raises(pkg.CapabilityError) as e:
        paged.fp8_paged_prefill(q, kc, vc, idx, page_size=16)
    assert e.value.field == "page_size" and isinstance(e.value, ValueError)
    with pytest.raises(ValueError, match="positions per page"):
        paged.fp8_paged_prefill(q, kc, vc, idx, page_size=1)


def test_rejects_non_causal_and_quantised_pools(pkg, paged):
    q, kc, vc, idx = _req()
    with pytest.raises(pkg.CapabilityError) as e:
        paged.fp8_paged_prefill(q, kc, vc, idx, causal=False)
    assert e.value.field == "mask"
    q, kc, vc, idx = _req(dtype=torch.float8_e4m3fn)
    with pytest.raises(pkg.CapabilityError) as e:
        paged.fp8_paged_prefill(q, kc, vc, idx)
    assert e.value.field == "kv_dtype"


def test_rejects_wrong_ranks(paged):
    q, kc, vc, idx = _req()
    with pytest.raises(ValueError, match="3-D"):
        paged.fp8_paged_prefill(q[0], kc, vc, idx)
    with pytest.raises(ValueError, match="paged_k_cache must be a 4-D"):
        paged.fp8_paged_prefill(q, kc[:, 0], vc, idx)
    with pytest.raises(ValueError, match="paged_v_cache must be a 4-D"):
        paged.fp8_paged_prefill(q, kc, vc[:, 0], idx)
    with pytest.raises(ValueError, match="kv_indices"):
        paged.fp8_paged_prefill(q, kc, vc, idx[None])


def test_more_queries_than_keys_is_the_operators_prefix_error(paged):
    q, kc, vc, idx = _req(qo=40, kv=32)
    with pytest.raises(ValueError, match="prefix"):
        paged.fp8_paged_prefill(q, kc, vc, idx)


def test_cpu_tensors_have_no_path(paged):
    q, kc, vc, idx = _req()
    with pytest.raises(RuntimeError, match="no CPU path"):
        paged.fp8_paged_prefill(q, kc, vc, idx)
