"""SGLang prefill attention backend over the sm_100a operator.

Mirror of the reference's `FP8PrefillAttnBackend`
(engines/sglang/integration/fp8_prefill/backend.py:87-291): a subclass of SGLang's FlashInfer
backend that overrides `forward_extend` only.  Pure-EXTEND forwards whose every request and whose
layer qualify run the fused FP8 operator of this package; everything else goes to the inherited
implementation with its metadata untouched.

What is kept from the reference, by name and meaning:
  * the class name, `init_forward_metadata`, `_layer_supported`, `_batch_qualifies`,
    `forward_extend(q, k, v, layer, forward_batch, save_kv_cache=True)` (:127-154, :158-184, :205-291);
  * the metadata-time snapshot: page rows and lengths are copied into owned tensors inside
    `init_forward_metadata`, and the layer-time path reads only that copy, because the overlap
    scheduler may rewrite `req_to_token` afterwards (:127-154);
  * pool write-through before the operator runs, so prefix and chunk are read uniformly from the
    pool (:226-231);
  * the environment knobs `SGLANG_FP8_PREFILL_DISABLE`, `_MIN_TOKENS` (8192), `_MIN_EXTEND` (0),
    `_K_CENTER`, `_HADAMARD`, `_QK`, `_BF16_HEADS`, `_DEBUG` (:93-113).

What differs:
  * `_BF16_HEADS` non-empty makes every forward take the inherited path, with the reason logged
    once (the bf16-PV lane is not on the declared surface and is not built); `_QK` accepts "int8"
    (default, as in the reference) and "fp8", anything else is treated the same way.
  * requests whose head counts are outside the declared capability surface (for example a
    tensor-parallel shard with 6:1 heads) take the inherited path instead of raising;
  * the per-request Python loop of three calls (:267-289) is one `prefill_extend_batch` call on the
    native batched entry (four launches for the whole forward, lengths and page rows in a device
    table) that writes each request's rows of the output in place; the batch workspace grows when a
    forward needs more, as the reference's per-backend workspace does;
  * a query that is not BF16, or a pool that is neither BF16 nor FP16, takes the inherited path
    before anything is written to the pool (the reference's preprocessing accepts any float type;
    this operator's contract is BF16 queries).
  * `register_backend(register)` is the registration the reference's installer appends to SGLang's
    backend registry (engines/sglang/integration/fp8_prefill/install.py:56-69), as a function.

SGLang is imported only when `FP8PrefillAttnBackend` is first asked for; a harness without SGLang
builds the class over its own base with `make_backend_class`.
"""
from __future__ import annotations

import logging
import os
from dataclasses import dataclass
from typing import Mapping, Optional, Sequence

from .capability import V1_CAPABILITY, CapabilityError, check_supported

HEAD_DIM = 256

logger = logging.getLogger(__name__)

__all__ = ["BackendSettings", "ExtendSnapshot", "make_backend_class", "register_backend", "FP8PrefillAttnBackend"]

BACKEND_NAME = "fp8_prefill"


@dataclass(frozen=True)
class BackendSettings:
    """The environment knobs, read once at construction (reference backend.py:93-113)."""
    disable: bool = False
    min_tokens: int = 8192
    min_extend: int = 0
    center_k: bool = True
    rotate: bool = True
    qk: str = "int8"
    bf16_heads: str = ""
    debug: bool = False

    @classmethod
    def from_env(cls, env: Optional[Mapping[str, str]] = None) -> "BackendSettings":
        env = os.environ if env is None else env
        return cls(
            disable=env.get("SGLANG_FP8_PREFILL_DISABLE") == "1",
            min_tokens=int(env.get("SGLANG_FP8_PREFILL_MIN_TOKENS", "8192")),
            min_extend=int(env.get("SGLANG_FP8_PREFILL_MIN_EXTEND", "0")),
            center_k=env.get("SGLANG_FP8_PREFILL_K_CENTER", "1") != "0",
            rotate=env.get("SGLANG_FP8_PREFILL_HADAMARD", "1") != "0",
            qk=env.get("SGLANG_FP8_PREFILL_QK", "int8").strip().lower(),
            bf16_heads=env.get("SGLANG_FP8_PREFILL_BF16_HEADS", "").strip(),
            debug=env.get("SGLANG_FP8_PREFILL_DEBUG") == "1",
        )

    def unbuilt_mode(self) -> Optional[str]:
        """Why the configured operator variant cannot run here, or None."""
        if self.qk not in ("int8", "fp8"):
            return f"SGLANG_FP8_PREFILL_QK={self.qk!r}: the QK operand type is int8 or fp8"
        if self.bf16_heads:
            return "SGLANG_FP8_PREFILL_BF16_HEADS is set: the bf16-PV lane is not built"
        return None


@dataclass(frozen=True)
class ExtendSnapshot:
    """Owned copy of what the scheduler said at metadata time (reference backend.py:139-153)."""
    prefix_lens: tuple
    extend_lens: tuple
    page_rows: tuple          # one int64 tensor [prefix + extend] per request, cloned

    def __len__(self) -> int:
        return len(self.prefix_lens)


def _is(value, *choices) -> bool:
    return any(value is c or value == c for c in choices)


def make_backend_class(base: type, extend_mode: object, *, name: str = "FP8PrefillAttnBackend") -> type:
    """Build the backend class over `base` (SGLang's `FlashInferAttnBackend`, or a stand-in with
    the same three members: `__init__(model_runner, ...)`, `init_forward_metadata(forward_batch)`,
    `forward_extend(q, k, v, layer, forward_batch, save_kv_cache=...)`).  `extend_mode` is the value
    `forward_batch.forward_mode` has on a pure EXTEND forward (`ForwardMode.EXTEND`)."""

    class _Backend(base):
        """FlashInfer everywhere, except qualifying EXTEND forwards, which run the fused FP8
        prefill operator."""

        def __init__(self, model_runner, *args, **kwargs):
            super().__init__(model_runner, *args, **kwargs)
            self._settings = BackendSettings.from_env()
            self._page_size = model_runner.server_args.page_size
            self._kv_cache_quantized = bool(
                getattr(model_runner.token_to_kv_pool, "is_quantized_kv_cache", False))
            self._fp8_snapshot: Optional[ExtendSnapshot] = None
            self._batch_ws = None
            self._unbuilt = self._settings.unbuilt_mode()
            self._last_decline: Optional[str] = None
            if self._settings.disable:
                logger.info("[fp8_prefill] disabled by SGLANG_FP8_PREFILL_DISABLE")
            elif self._unbuilt:
                logger.warning("[fp8_prefill] every forward takes the inherited path: %s", self._unbuilt)
            else:
                logger.info("[fp8_prefill] enabled: qk=%s min_tokens=%d min_extend=%d page_size=%d",
                            self._settings.qk, self._settings.min_tokens, self._settings.min_extend,
                            self._page_size)

        # ---- metadata time -------------------------------------------------------------
        def init_forward_metadata(self, forward_batch):
            ret = super().init_forward_metadata(forward_batch)
            self._fp8_snapshot = None
            prefix = getattr(forward_batch, "extend_prefix_lens_cpu", None)
            extend = getattr(forward_batch, "extend_seq_lens_cpu", None)
            if (self._settings.disable or self._unbuilt or prefix is None or extend is None
                    or not _is(forward_batch.forward_mode, extend_mode)):
                return ret
            import torch

            prefix = tuple(int(x) for x in prefix)
            extend = tuple(int(x) for x in extend)
            rows = forward_batch.req_pool_indices.tolist()
            table = self.req_to_token_pool.req_to_token
            pages = tuple(table[row, : p + e].to(torch.int64).clone()
                          for row, p, e in zip(rows, prefix, extend))
            self._fp8_snapshot = ExtendSnapshot(prefix, extend, pages)
            return ret

        # ---- eligibility ---------------------------------------------------------------
        def _layer_decline(self, layer) -> Optional[str]:
            if layer.head_dim != HEAD_DIM or getattr(layer, "v_head_dim", HEAD_DIM) != HEAD_DIM:
                return "head_dim is not 256"
            if layer.tp_q_head_num % max(layer.tp_k_head_num, 1) != 0:
                return "q heads not a multiple of kv heads"
            if layer.logit_cap not in (0, 0.0, None):
                return "logit cap"
            if getattr(layer, "sliding_window_size", None) not in (None, -1):
                return "sliding window"
            if layer.is_cross_attention:
                return "cross attention"
            try:
                check_supported(head_dim=layer.head_dim, q_heads=layer.tp_q_head_num,
                                kv_heads=layer.tp_k_head_num, page_size=self._page_size,
                                mode="extend", mask="bottom_right_causal", kv_dtype="bfloat16",
                                capability=V1_CAPABILITY)
            except CapabilityError as exc:
                return f"outside the declared surface: {exc}"
            return None

        def _batch_decline(self, forward_batch) -> Optional[str]:
            s = self._settings
            if s.disable:
                return "disabled"
            if self._unbuilt:
                return self._unbuilt
            if self._kv_cache_quantized:
                return "quantised KV pool"
            if self._page_size != 1:
                return "page size is not 1"
            if not _is(forward_batch.forward_mode, extend_mode):
                return "not a pure EXTEND forward"
            snap = self._fp8_snapshot
            if snap is None:
                return "no metadata snapshot"
            multi_item = getattr(getattr(self, "forward_metadata", None), "multi_item_params", None)
            if multi_item is not None and multi_item.is_enabled():
                return "multi-item scoring"
            for p, e in zip(snap.prefix_lens, snap.extend_lens):
                if p + e < s.min_tokens:
                    return f"request of {p + e} tokens is below SGLANG_FP8_PREFILL_MIN_TOKENS"
                if e < s.min_extend:
                    return f"extend of {e} tokens is below SGLANG_FP8_PREFILL_MIN_EXTEND"
            return None

        def _layer_supported(self, layer) -> bool:
            return self._layer_decline(layer) is None

        def _batch_qualifies(self, forward_batch) -> bool:
            return self._batch_decline(forward_batch) is None

        # ---- forward -------------------------------------------------------------------
        def forward_extend(self, q, k, v, layer, forward_batch, save_kv_cache=True):
            reason = self._batch_decline(forward_batch) or self._layer_decline(layer)
            if reason is not None:
                if reason != self._last_decline and self._settings.debug:
                    logger.info("[fp8_prefill] inherited path: %s", reason)
                self._last_decline = reason
                return super().forward_extend(q, k, v, layer, forward_batch, save_kv_cache=save_kv_cache)
            import torch

            from . import ops
            from .quant import FP8PrefillBatchWorkspace

            heads = layer.tp_q_head_num
            k_pool = self.token_to_kv_pool.get_key_buffer(layer.layer_id)
            v_pool = self.token_to_kv_pool.get_value_buffer(layer.layer_id)
            # operand types are checked before the pool write-through: after it the forward could no
            # longer be handed to the inherited path
            reason = None
            if q.dtype != torch.bfloat16:
                reason = f"query dtype {q.dtype} is not bfloat16"
            elif k_pool.dtype not in (torch.bfloat16, torch.float16) or v_pool.dtype != k_pool.dtype:
                reason = f"pool dtype {k_pool.dtype} is neither bfloat16 nor float16"
            elif not (k_pool.is_contiguous() and v_pool.is_contiguous()):
                reason = "pool buffers are not contiguous"
            if reason is not None:
                if reason != self._last_decline and self._settings.debug:
                    logger.info("[fp8_prefill] inherited path: %s", reason)
                self._last_decline = reason
                return super().forward_extend(q, k, v, layer, forward_batch, save_kv_cache=save_kv_cache)
            self._last_decline = None

            # 1. the chunk's K/V go into the paged pool first; the operator then reads prefix and
            #    chunk alike from the pool
            if k is not None and save_kv_cache:
                if v is None:
                    raise ValueError("forward_extend: k given without v")
                scales = self._kv_write_scales(layer) if hasattr(self, "_kv_write_scales") else (
                    getattr(layer, "k_scale", None), getattr(layer, "v_scale", None))
                self.token_to_kv_pool.set_kv_buffer(layer, forward_batch.out_cache_loc, k, v, *scales)

            q3 = q.view(-1, heads, HEAD_DIM)
            out = torch.empty_like(q3)

            # 2. one batched call; lengths and page rows come from the snapshot only
            snap = self._fp8_snapshot
            if sum(snap.extend_lens) != q3.shape[0]:
                raise ValueError(
                    f"forward_extend: q has {q3.shape[0]} rows but the metadata snapshot describes "
                    f"{sum(snap.extend_lens)}")
            requests, row0 = [], 0
            for p, e, pages in zip(snap.prefix_lens, snap.extend_lens, snap.page_rows):
                requests.append({"q": q3[row0:row0 + e], "k_pool": k_pool, "v_pool": v_pool,
                                 "idx": pages, "prefix": p, "out": out[row0:row0 + e]})
                row0 += e
            kv_total = sum(p + e for p, e in zip(snap.prefix_lens, snap.extend_lens))
            ws = self._batch_ws
            if (ws is None or ws.device != q.device or (ws.q_heads, ws.kv_heads) != (heads, layer.tp_k_head_num)
                    or not ws.admits(len(requests), kv_total, q3.shape[0])):
                # grow with headroom (eager use; a deployment that captures graphs reserves once)
                ws = FP8PrefillBatchWorkspace(
                    q.device, max_requests=max(len(requests), 8) * 2, max_total_kv_len=int(kv_total * 1.5) + 1024,
                    max_total_q_len=int(q3.shape[0] * 1.5) + 256, q_heads=heads, kv_heads=layer.tp_k_head_num)
                self._batch_ws = ws
            ops.prefill_extend_batch(requests, workspace=ws, sm_scale=layer.scaling,
                                     qk_i8=self._settings.qk == "int8", rotate=self._settings.rotate,
                                     center_k=self._settings.center_k)
            return out.view(-1, heads * HEAD_DIM)

    _Backend.__name__ = _Backend.__qualname__ = name
    return _Backend


def register_backend(register, *, name: str = BACKEND_NAME, backend_class: Optional[type] = None):
    """Register the backend factory under `name` with an attention-backend registry.

    `register` is the registry's decorator factory -- SGLang's `register_attention_backend` -- so that
    `register(name)(factory)` files the factory.  The factory refuses MLA models and forwards the
    runner's workspace policy unchanged, as the block the reference's installer appends to SGLang's
    registry does (engines/sglang/integration/fp8_prefill/install.py:56-69).  `backend_class`
    defaults to the class bound to the installed SGLang.  Returns the factory."""

    def create_fp8_prefill_backend(runner):
        if getattr(runner, "use_mla_backend", False):
            raise ValueError("fp8_prefill does not support MLA models.")
        cls = backend_class if backend_class is not None else __getattr__("FP8PrefillAttnBackend")
        return cls(runner, init_new_workspace=runner.init_new_workspace)

    register(name)(create_fp8_prefill_backend)
    return create_fp8_prefill_backend


_sglang_class: Optional[type] = None


def __getattr__(attr: str):
    """`FP8PrefillAttnBackend` bound to the installed SGLang, built on first access."""
    global _sglang_class
    if attr != "FP8PrefillAttnBackend":
        raise AttributeError(attr)
    if _sglang_class is None:
        try:
            from sglang.srt.layers.attention.flashinfer_backend import FlashInferAttnBackend
            from sglang.srt.model_executor.forward_batch_info import ForwardMode
        except ImportError as exc:
            raise ImportError(
                "FP8PrefillAttnBackend needs SGLang (sglang.srt.layers.attention.flashinfer_backend); "
                "without it, build the class over your own base with make_backend_class(base, extend_mode)"
            ) from exc
        _sglang_class = make_backend_class(FlashInferAttnBackend, ForwardMode.EXTEND)
    return _sglang_class
