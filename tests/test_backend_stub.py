"""The SGLang backend class against stand-ins for SGLang (no GPU, no SGLang): eligibility gates
and fallback routing, the metadata-time snapshot, pool write-through order, and what the batched
operator call receives (engines/sglang/integration/fp8_prefill/backend.py:127-291)."""
import pytest
import torch

import sglang_stubs as S


@pytest.fixture()
def backend_mod(pkg):
    from attn_kernel_lab_b200 import backend
    return backend


def _setup(backend_mod, monkeypatch, *, env=None, prefix=(9000, 8500), extend=(512, 300), page_size=1,
           quantized=False, layer=None):
    for key in ("DISABLE", "MIN_TOKENS", "MIN_EXTEND", "K_CENTER", "HADAMARD", "QK", "BF16_HEADS", "DEBUG"):
        monkeypatch.delenv("SGLANG_FP8_PREFILL_" + key, raising=False)
    for k, v in (env or {}).items():
        monkeypatch.setenv(k, v)
    cls = backend_mod.make_backend_class(S.BaseBackend, S.ForwardMode.EXTEND)
    dev = torch.device("cpu")
    pool = S.KVPool(32768, 4, 2, dev, quantized=quantized)
    total = [p + e for p, e in zip(prefix, extend)]
    table = torch.zeros(4, max(total) + 8, dtype=torch.int32)
    g = torch.Generator().manual_seed(5)
    perm = torch.randperm(32768, generator=g).to(torch.int32)
    at = 0
    for r, n in enumerate(total):
        table[r + 1, :n] = perm[at:at + n]          # request r lives in table row r + 1
        at += n
    runner = S.model_runner(pool, table, page_size)
    be = cls(runner)
    new_rows = torch.cat([table[r + 1, p:p + e] for r, (p, e) in enumerate(zip(prefix, extend))])
    fb = S.ForwardBatch(S.ForwardMode.EXTEND, list(prefix), list(extend),
                        torch.arange(1, len(prefix) + 1), new_rows)
    layer = layer or S.Layer(layer_id=1)
    tokens = sum(extend)
    q = torch.randn(tokens, layer.tp_q_head_num * 256, generator=g).to(torch.bfloat16)
    k = torch.randn(tokens, layer.tp_k_head_num * 256, generator=g).to(torch.bfloat16)
    v = torch.randn(tokens, layer.tp_k_head_num * 256, generator=g).to(torch.bfloat16)
    return be, fb, layer, (q, k, v), pool, table


class Recorder:
    def __init__(self):
        self.calls = []

    def __call__(self, requests, *, workspace, sm_scale=None, qk_i8=False, rotate=True, center_k=True, **kw):
        requests = list(requests)
        self.calls.append({"requests": requests, "workspace": workspace, "sm_scale": sm_scale,
                           "qk_i8": qk_i8, "rotate": rotate, "center_k": center_k})
        for i, r in enumerate(requests):
            r["out"].fill_(float(i + 1))
        return [r["out"] for r in requests]


def _patch_operator(backend_mod, monkeypatch):
    from attn_kernel_lab_b200 import ops, quant
    rec = Recorder()
    monkeypatch.setattr(ops, "prefill_extend_batch", rec)
    class FakeBatchWorkspace:
        """Stands in for the batch workspace: records what it was sized for, allocates nothing."""
        made = []

        def __init__(self, device, *, max_requests, max_total_kv_len, max_total_q_len, q_heads, kv_heads):
            self.device, self.q_heads, self.kv_heads = device, q_heads, kv_heads
            self.sizes = (max_requests, max_total_kv_len, max_total_q_len)
            FakeBatchWorkspace.made.append(self)

        def admits(self, n, kv, qlen):
            return n <= self.sizes[0] and kv <= self.sizes[1] and qlen <= self.sizes[2]

    monkeypatch.setattr(quant, "FP8PrefillBatchWorkspace", FakeBatchWorkspace)
    rec.workspace_class = FakeBatchWorkspace
    return rec


def test_qualifying_forward_runs_the_operator_from_the_snapshot(backend_mod, monkeypatch):
    be, fb, layer, (q, k, v), pool, table = _setup(backend_mod, monkeypatch)
    rec = _patch_operator(backend_mod, monkeypatch)
    assert be.init_forward_metadata(fb) == "base-metadata" and be.metadata_calls == 1
    snap = be._fp8_snapshot
    assert snap.prefix_lens == (9000, 8500) and snap.extend_lens == (512, 300)
    want_rows = [table[1, :9512].long().clone(), table[2, :8800].long().clone()]
    # the scheduler rewrites its buffers after metadata time: the layer-time path must not see it
    table.zero_()
    fb.extend_prefix_lens_cpu[:] = [1, 1]
    fb.extend_seq_lens_cpu[:] = [1, 1]
    out = be.forward_extend(q, k, v, layer, fb)
    assert be.fallback_calls == []
    assert pool.writes == [(1, 812)], "the chunk is written through to the pool, once, before the operator"
    (call,) = rec.calls
    assert call["sm_scale"] == layer.scaling and call["rotate"] and call["center_k"]
    assert call["qk_i8"] is True, "INT8 QK is the default operand type, as in the reference"
    ws = call["workspace"]
    assert isinstance(ws, rec.workspace_class) and (ws.q_heads, ws.kv_heads) == (24, 4)
    assert ws.admits(2, 9512 + 8800, 812), "sized for this forward, with headroom"
    be.forward_extend(q, k, v, layer, fb, save_kv_cache=False)
    assert rec.calls[-1]["workspace"] is ws and len(rec.workspace_class.made) == 1, "the workspace is kept between layers"
    del rec.calls[-1]
    r0, r1 = call["requests"]
    assert r0["prefix"] == 9000 and r1["prefix"] == 8500
    assert torch.equal(r0["idx"], want_rows[0]) and torch.equal(r1["idx"], want_rows[1])
    assert r0["idx"].dtype == torch.int64
    assert r0["q"].shape == (512, 24, 256) and r1["q"].shape == (300, 24, 256)
    assert r0["k_pool"] is pool.k[1] and r0["v_pool"] is pool.v[1]
    assert out.shape == q.shape
    o3 = out.view(-1, 24, 256)
    assert (o3[:512] == 1).all() and (o3[512:] == 2).all(), "each request's rows are written in place"
    # the written-through rows are what the pool now holds at out_cache_loc
    assert torch.equal(pool.k[1][fb.out_cache_loc.long()].view(812, -1), k)


def test_operand_types_outside_the_contract_decline_before_the_pool_write(backend_mod, monkeypatch):
    """An FP16-activation model (or an FP32 pool) must take the inherited path, and must do so before
    the chunk is written through: afterwards the forward could not be handed over any more."""
    be, fb, layer, (q, k, v), pool, _ = _setup(backend_mod, monkeypatch)
    rec = _patch_operator(backend_mod, monkeypatch)
    be.init_forward_metadata(fb)
    out = be.forward_extend(q.to(torch.float16), k, v, layer, fb)
    assert rec.calls == [] and pool.writes == [] and be.fallback_calls == [(layer.layer_id, True)]
    assert (out == -7).all()
    pool.k[1] = pool.k[1].float()
    pool.v[1] = pool.v[1].float()
    be.forward_extend(q, k, v, layer, fb)
    assert rec.calls == [] and pool.writes == [] and len(be.fallback_calls) == 2


def test_register_backend_files_the_factory_under_the_reference_name(backend_mod):
    registry = {}

    def register_attention_backend(name):          # the shape of SGLang's registry decorator
        def deco(fn):
            registry[name] = fn
            return fn
        return deco

    class Cls:
        def __init__(self, runner, **kw):
            self.runner, self.kw = runner, kw

    factory = backend_mod.register_backend(register_attention_backend, backend_class=Cls)
    assert registry == {"fp8_prefill": factory}
    runner = type("Runner", (), {"use_mla_backend": False, "init_new_workspace": "policy"})()
    made = registry["fp8_prefill"](runner)
    assert isinstance(made, Cls) and made.runner is runner and made.kw == {"init_new_workspace": "policy"}
    runner.use_mla_backend = True
    with pytest.raises(ValueError, match="MLA"):
        registry["fp8_prefill"](runner)


def test_save_kv_cache_false_skips_the_write(backend_mod, monkeypatch):
    be, fb, layer, (q, k, v), pool, _ = _setup(backend_mod, monkeypatch)
    _patch_operator(backend_mod, monkeypatch)
    be.init_forward_metadata(fb)
    be.forward_extend(q, k, v, layer, fb, save_kv_cache=False)
    assert pool.writes == []


@pytest.mark.parametrize("why, kwargs", [
    ("disabled", dict(env={"SGLANG_FP8_PREFILL_DISABLE": "1"})),
    ("unknown QK operand type", dict(env={"SGLANG_FP8_PREFILL_QK": "fp4"})),
    ("bf16-PV lane is not built", dict(env={"SGLANG_FP8_PREFILL_BF16_HEADS": "0,3"})),
    ("short request", dict(prefix=(9000, 100), extend=(512, 300))),
    ("short extend", dict(env={"SGLANG_FP8_PREFILL_MIN_EXTEND": "400"})),
    ("page size", dict(page_size=16)),
    ("quantised pool", dict(quantized=True)),
    ("head dim", dict(layer=S.Layer(head_dim=128, v_head_dim=128))),
    ("logit cap", dict(layer=S.Layer(logit_cap=30.0))),
    ("sliding window", dict(layer=S.Layer(sliding_window_size=4096))),
    ("cross attention", dict(layer=S.Layer(is_cross_attention=True))),
    ("heads outside the surface", dict(layer=S.Layer(tp_q_head_num=6, tp_k_head_num=1))),
])
def test_everything_else_takes_the_inherited_path(backend_mod, monkeypatch, why, kwargs):
    be, fb, layer, (q, k, v), pool, _ = _setup(backend_mod, monkeypatch, **kwargs)
    rec = _patch_operator(backend_mod, monkeypatch)
    be.init_forward_metadata(fb)
    out = be.forward_extend(q, k, v, layer, fb)
    assert rec.calls == [], why
    assert be.fallback_calls == [(layer.layer_id, True)], why
    assert (out == -7).all()
    assert pool.writes == [], "the inherited path does its own pool write"


def test_other_forward_modes_and_missing_metadata_fall_back(backend_mod, monkeypatch):
    be, fb, layer, (q, k, v), _, _ = _setup(backend_mod, monkeypatch)
    rec = _patch_operator(backend_mod, monkeypatch)
    be.forward_extend(q, k, v, layer, fb)                 # no init_forward_metadata yet
    assert len(be.fallback_calls) == 1 and rec.calls == []
    fb.forward_mode = S.ForwardMode.MIXED
    be.init_forward_metadata(fb)
    assert be._fp8_snapshot is None
    be.forward_extend(q, k, v, layer, fb)
    assert len(be.fallback_calls) == 2 and rec.calls == []
    fb.forward_mode = S.ForwardMode.EXTEND
    be.init_forward_metadata(fb)
    be.forward_metadata.multi_item_params = type("M", (), {"is_enabled": lambda self: True})()
    be.forward_extend(q, k, v, layer, fb)
    assert len(be.fallback_calls) == 3 and rec.calls == []
    assert not be._batch_qualifies(fb) and be._layer_supported(layer)


def test_knobs_reach_the_operator(backend_mod, monkeypatch):
    be, fb, layer, (q, k, v), _, _ = _setup(
        backend_mod, monkeypatch, env={"SGLANG_FP8_PREFILL_K_CENTER": "0", "SGLANG_FP8_PREFILL_HADAMARD": "0",
                                       "SGLANG_FP8_PREFILL_QK": "fp8",
                                       "SGLANG_FP8_PREFILL_MIN_TOKENS": "100"})
    rec = _patch_operator(backend_mod, monkeypatch)
    be.init_forward_metadata(fb)
    be.forward_extend(q, k, v, layer, fb)
    (call,) = rec.calls
    assert call["rotate"] is False and call["center_k"] is False and call["qk_i8"] is False
    assert isinstance(call["workspace"], rec.workspace_class)


def test_row_count_mismatch_is_an_error_not_a_silent_slice(backend_mod, monkeypatch):
    be, fb, layer, (q, k, v), _, _ = _setup(backend_mod, monkeypatch)
    _patch_operator(backend_mod, monkeypatch)
    be.init_forward_metadata(fb)
    with pytest.raises(ValueError, match="metadata snapshot"):
        be.forward_extend(q[:-1], k[:-1], v[:-1], layer, fb, save_kv_cache=False)


def test_module_attribute_needs_sglang(backend_mod):
    try:
        import sglang  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError, match="make_backend_class"):
            backend_mod.FP8PrefillAttnBackend
