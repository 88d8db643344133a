"""Stand-ins for the SGLang objects the prefill backend touches, so that the backend class can
be exercised without SGLang: a base backend that records what reaches it, a page-size-1 KV pool,
the request-to-token table, a forward batch and an attention layer
(the members used are those of engines/sglang/integration/fp8_prefill/backend.py:116-119,
139-153, 158-166, 226-238)."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from types import SimpleNamespace

import torch


class ForwardMode(enum.Enum):
    EXTEND = 1
    DECODE = 2
    MIXED = 3
    TARGET_VERIFY = 4


class KVPool:
    """[pool, kv_heads, 256] K and V planes per layer; rows written through `set_kv_buffer`."""

    def __init__(self, slots: int, kv_heads: int, layers: int, device, dtype=torch.bfloat16, quantized=False):
        self.k = [torch.zeros(slots, kv_heads, 256, dtype=dtype, device=device) for _ in range(layers)]
        self.v = [torch.zeros(slots, kv_heads, 256, dtype=dtype, device=device) for _ in range(layers)]
        self.is_quantized_kv_cache = quantized
        self.writes = []

    def set_kv_buffer(self, layer, loc, k, v, k_scale=None, v_scale=None):
        self.writes.append((layer.layer_id, int(loc.numel())))
        heads = self.k[layer.layer_id].shape[1]
        self.k[layer.layer_id][loc.long()] = k.view(-1, heads, 256).to(self.k[layer.layer_id].dtype)
        self.v[layer.layer_id][loc.long()] = v.view(-1, heads, 256).to(self.v[layer.layer_id].dtype)

    def get_key_buffer(self, layer_id):
        return self.k[layer_id]

    def get_value_buffer(self, layer_id):
        return self.v[layer_id]


class BaseBackend:
    """What FlashInferAttnBackend is to the class under test: it owns the pools, builds the
    metadata and has the fallback `forward_extend`."""

    def __init__(self, model_runner, *args, **kwargs):
        self.req_to_token_pool = model_runner.req_to_token_pool
        self.token_to_kv_pool = model_runner.token_to_kv_pool
        self.forward_metadata = SimpleNamespace(multi_item_params=None)
        self.metadata_calls = 0
        self.fallback_calls = []

    def init_forward_metadata(self, forward_batch):
        self.metadata_calls += 1
        return "base-metadata"

    def forward_extend(self, q, k, v, layer, forward_batch, save_kv_cache=True):
        self.fallback_calls.append((layer.layer_id, save_kv_cache))
        return torch.full_like(q, -7.0)

    def _kv_write_scales(self, layer):
        return (None, None)


@dataclass
class Layer:
    layer_id: int = 0
    head_dim: int = 256
    v_head_dim: int = 256
    tp_q_head_num: int = 24
    tp_k_head_num: int = 4
    logit_cap: float = 0.0
    sliding_window_size: int = -1
    is_cross_attention: bool = False
    scaling: float = 1.0 / 16.0


@dataclass
class ForwardBatch:
    forward_mode: ForwardMode
    extend_prefix_lens_cpu: list
    extend_seq_lens_cpu: list
    req_pool_indices: torch.Tensor
    out_cache_loc: torch.Tensor
    extra: dict = field(default_factory=dict)


def model_runner(pool: KVPool, req_to_token: torch.Tensor, page_size: int = 1):
    return SimpleNamespace(server_args=SimpleNamespace(page_size=page_size), token_to_kv_pool=pool,
                           req_to_token_pool=SimpleNamespace(req_to_token=req_to_token))
