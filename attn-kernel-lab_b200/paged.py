"""FlashInfer-shaped entry: one request over a paged NHD KV cache.

Same call shape as the reference's upstream-facing shim
(upstream/pr-draft/tests/attention/flashinfer_shim.py:198-268): `q` [qo_len, num_qo_heads, 256]
BF16, `paged_k_cache` / `paged_v_cache` [num_pages, page_size, num_kv_heads, 256] (NHD),
`kv_indices` [kv_len] page ids in position order with the cached prefix first.  The number of
cached positions is implied: `prefix = kv_len - qo_len`, i.e. the bottom-right causal mask.

The two axes that a reshape of the cache would otherwise reinterpret silently -- `page_size` and the
mask -- are checked against the declared surface before any tensor is touched, so that
`page_size=16` or `causal=False` is a `CapabilityError` (a `ValueError`) and never a mis-shaped read.
"""
from __future__ import annotations

from .capability import V1_CAPABILITY, OperatorCapability, check_supported

__all__ = ["fp8_paged_prefill"]


def _is_tensor(x) -> bool:
    return hasattr(x, "dim") and hasattr(x, "shape") and hasattr(x, "dtype")


def fp8_paged_prefill(q, paged_k_cache, paged_v_cache, kv_indices, *, page_size: int = 1,
                      causal: bool = True, sm_scale=None, out=None, return_lse: bool = False,
                      workspace_buffer=None, capability: OperatorCapability = V1_CAPABILITY):
    """Returns `out` [qo_len, num_qo_heads, 256] BF16 (the caller's `out` when given), or
    `(out, lse)` with base-2 `lse` [qo_len, num_qo_heads] FP32 when `return_lse`.

    `workspace_buffer` is an `FP8PrefillWorkspace` (named after the upstream argument); with a
    planned workspace the call allocates nothing but `out`.  Everything else -- validation order,
    error types, stream semantics -- is `prefill_extend`'s."""
    if not _is_tensor(q) or q.dim() != 3:
        raise ValueError("q must be a 3-D [qo_len, num_qo_heads, head_dim] tensor")
    for name, cache in (("paged_k_cache", paged_k_cache), ("paged_v_cache", paged_v_cache)):
        if not _is_tensor(cache) or cache.dim() != 4:
            got = f"{cache.dim()}-D" if _is_tensor(cache) else type(cache).__name__
            raise ValueError(f"{name} must be a 4-D [num_pages, page_size, num_kv_heads, head_dim] "
                             f"NHD tensor, got {got}")
    if not _is_tensor(kv_indices) or kv_indices.dim() != 1:
        raise ValueError("kv_indices must be a 1-D tensor of page ids in position order")

    check_supported(
        head_dim=int(q.shape[2]), q_heads=int(q.shape[1]), kv_heads=int(paged_k_cache.shape[2]),
        page_size=int(page_size), mode="extend",
        mask="bottom_right_causal" if causal else "noncausal",
        kv_dtype=str(paged_k_cache.dtype).rsplit(".", 1)[-1], return_lse=bool(return_lse),
        capability=capability)
    if int(paged_k_cache.shape[1]) != int(page_size) or int(paged_v_cache.shape[1]) != int(page_size):
        raise ValueError(f"the caches hold {int(paged_k_cache.shape[1])} positions per page, "
                         f"page_size says {int(page_size)}")

    from . import ops

    # page_size == 1 from here on: a page is a position, and the page table is the index list
    k_pool = paged_k_cache[:, 0]
    v_pool = paged_v_cache[:, 0]
    prefix = int(kv_indices.numel()) - int(q.shape[0])
    return ops.prefill_extend(q, k_pool, v_pool, kv_indices, prefix, workspace=workspace_buffer,
                              out=out, sm_scale=sm_scale, return_lse=return_lse, capability=capability)
