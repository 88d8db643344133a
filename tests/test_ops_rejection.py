"""Every declared-surface rejection, on CPU, with no native call.

Same contract as the reference's tests/test_ops_rejection.py: each out-of-surface request
raises `CapabilityError` (a `ValueError`) naming the field, with a message a caller can act
on, and validation never reaches the native library -- `kernel.load` is replaced by a tripwire.
"""
import pytest
import torch

Q_LEN, Q_HEADS, KV_HEADS, HEAD_DIM, KV_LEN = 8, 24, 4, 256, 32
PREFIX = KV_LEN - Q_LEN


class _LoadAttempted(RuntimeError):
    pass


@pytest.fixture(autouse=True)
def no_native_load(pkg, monkeypatch):
    from attn_kernel_lab_b200 import kernel as kernel_mod

    def trip(*a, **k):
        raise _LoadAttempted("kernel.load() must not be reached by validation")

    monkeypatch.setattr(kernel_mod, "load", trip)


def _call(**over):
    call = dict(
        q=torch.zeros((Q_LEN, Q_HEADS, HEAD_DIM), dtype=torch.bfloat16),
        k_pool=torch.zeros((KV_LEN, KV_HEADS, HEAD_DIM), dtype=torch.bfloat16),
        v_pool=torch.zeros((KV_LEN, KV_HEADS, HEAD_DIM), dtype=torch.bfloat16),
        idx=torch.arange(KV_LEN, dtype=torch.int64),
        prefix=PREFIX,
    )
    call.update(over)
    return call


def _geometry(*, q_heads=Q_HEADS, kv_heads=KV_HEADS, head_dim=HEAD_DIM):
    return _call(
        q=torch.zeros((Q_LEN, q_heads, head_dim), dtype=torch.bfloat16),
        k_pool=torch.zeros((KV_LEN, kv_heads, head_dim), dtype=torch.bfloat16),
        v_pool=torch.zeros((KV_LEN, kv_heads, head_dim), dtype=torch.bfloat16),
    )


def _fp8_pool():
    pool = torch.zeros((KV_LEN, KV_HEADS, HEAD_DIM), dtype=torch.float8_e4m3fn)
    return _call(k_pool=pool, v_pool=pool.clone())


CASES = [
    (lambda: _geometry(head_dim=128), {}, "head_dim", r"head_dim=128 is outside the declared support surface"),
    (lambda: _geometry(head_dim=64), {}, "head_dim", r"head_dim=64 is outside the declared support surface"),
    (lambda: _geometry(q_heads=8, kv_heads=4), {}, "q_heads", r"q_heads=8 is outside the declared support surface"),
    (lambda: _geometry(q_heads=24, kv_heads=2), {}, "kv_heads", r"kv_heads=2 is outside the declared support surface"),
    (_fp8_pool, {}, "kv_dtype", r"kv_dtype='float8_e4m3fn' is outside the declared support surface"),
    (lambda: _call(q=torch.zeros((Q_LEN, Q_HEADS * HEAD_DIM), dtype=torch.bfloat16)), {}, "q", r"q must be 3-D"),
    (lambda: _call(q=[1, 2, 3]), {}, "q", r"q must be a torch.Tensor, got list"),
    (lambda: _call(q=torch.zeros((Q_LEN, Q_HEADS, 2 * HEAD_DIM), dtype=torch.bfloat16)[:, :, ::2]), {}, "q", r"q must be contiguous"),
    (lambda: _call(q=torch.zeros((Q_LEN, Q_HEADS, HEAD_DIM), dtype=torch.float16)), {}, "q", r"q dtype must be bfloat16"),
    (lambda: _call(q=torch.zeros((0, Q_HEADS, HEAD_DIM), dtype=torch.bfloat16), prefix=0), {}, "q_len", r"q_len must be >= 1"),
    (lambda: _call(k_pool=torch.zeros((KV_LEN, KV_HEADS * HEAD_DIM), dtype=torch.bfloat16)), {}, "k_pool", r"k_pool must be 3-D"),
    (lambda: _call(k_pool=torch.zeros((KV_LEN, KV_HEADS, 128), dtype=torch.bfloat16),
                   v_pool=torch.zeros((KV_LEN, KV_HEADS, 128), dtype=torch.bfloat16)), {}, "k_pool",
     r"k_pool head_dim 128 must equal q head_dim 256"),
    (lambda: _call(v_pool=torch.zeros((KV_LEN + 1, KV_HEADS, HEAD_DIM), dtype=torch.bfloat16)), {}, "v_pool", r"v_pool shape .* must equal k_pool shape"),
    (lambda: _call(v_pool=torch.zeros((KV_LEN, KV_HEADS, HEAD_DIM), dtype=torch.float16)), {}, "v_pool", r"v_pool dtype float16 must equal k_pool dtype bfloat16"),
    (lambda: _call(idx=torch.arange(KV_LEN).view(2, -1)), {}, "idx", r"idx must be 1-D"),
    (lambda: _call(idx=torch.arange(KV_LEN, dtype=torch.int16)), {}, "idx", r"idx dtype must be int64"),
    (lambda: _call(idx=torch.arange(0, dtype=torch.int64), prefix=0), {}, "idx", r"idx must name at least one kv position"),
    (lambda: _call(idx=torch.arange(KV_LEN, dtype=torch.int64, device="meta")), {}, "idx", r"idx is on meta but q is on cpu"),
    (lambda: _call(prefix=-1), {}, "prefix", r"prefix=-1 is outside \[0, kv_len - q_len\]"),
    (lambda: _call(prefix=KV_LEN), {}, "prefix", r"prefix=32 is outside \[0, kv_len - q_len\] = \[0, 24\]"),
    (lambda: _call(prefix=3.0), {}, "prefix", r"prefix must be a Python int, got float"),
    (lambda: _call(prefix=True), {}, "prefix", r"prefix must be a Python int, got bool"),
    (_call, {"sm_scale": 0.0}, "sm_scale", r"sm_scale must be positive and finite"),
    (_call, {"sm_scale": float("inf")}, "sm_scale", r"sm_scale must be positive and finite"),
    (_call, {"sm_scale": "0.1"}, "sm_scale", r"sm_scale must be a real number or None, got str"),
    (_call, {"out": torch.zeros((Q_LEN, Q_HEADS, 128), dtype=torch.bfloat16)}, "out", r"out shape .* must equal q shape"),
    (_call, {"out": torch.zeros((Q_LEN, Q_HEADS, HEAD_DIM), dtype=torch.float32)}, "out", r"out dtype must be bfloat16"),
    (_call, {"out": torch.zeros((Q_LEN, Q_HEADS, 2 * HEAD_DIM), dtype=torch.bfloat16)[:, :, ::2]}, "out", r"out must be contiguous"),
    (_call, {"out": torch.zeros((Q_LEN, Q_HEADS, HEAD_DIM), dtype=torch.bfloat16, device="meta")}, "out", r"out is on meta but q is on cpu"),
    (_call, {"out": "buffer"}, "out", r"out must be a torch.Tensor or None, got str"),
    (_call, {"lse_out": torch.zeros((Q_LEN, Q_HEADS), dtype=torch.float32)}, "lse_out", r"lse_out was supplied but return_lse=False"),
    (_call, {"return_lse": True, "lse_out": torch.zeros((Q_LEN, Q_HEADS + 1), dtype=torch.float32)}, "lse_out", r"lse_out shape .* must be \(8, 24\)"),
    (_call, {"return_lse": True, "lse_out": torch.zeros((Q_LEN, Q_HEADS), dtype=torch.float16)}, "lse_out", r"lse_out dtype must be float32"),
    (_call, {"return_lse": True, "lse_out": torch.zeros((Q_LEN, 2 * Q_HEADS), dtype=torch.float32)[:, ::2]}, "lse_out", r"lse_out must be contiguous"),
    (_call, {"workspace": object()}, "workspace", r"workspace must be .*FP8PrefillWorkspace or None, got builtins.object"),
]


@pytest.mark.parametrize("build,kwargs,field,match", CASES, ids=[f"{i:02d}-{c[2]}" for i, c in enumerate(CASES)])
def test_rejected_before_any_device_work(pkg, build, kwargs, field, match):
    with pytest.raises(pkg.CapabilityError, match=match) as info:
        pkg.prefill_extend(**build(), **kwargs)
    assert info.value.field == field
    assert isinstance(info.value, ValueError)


def test_out_must_not_alias_q(pkg):
    call = _call()
    with pytest.raises(pkg.CapabilityError, match=r"out must not overlap q storage") as info:
        pkg.prefill_extend(**call, out=call["q"])
    assert info.value.field == "out"


def test_int8_qk_is_accepted_and_reaches_the_device_check(pkg):
    """Both QK operand types pass validation; on CPU tensors the call then stops where every
    accepted request stops, at the missing device (there is no CPU path)."""
    for mode in (True, False):
        with pytest.raises(RuntimeError, match="no CPU path"):
            pkg.prefill_extend(**_call(), qk_i8=mode)
    with pytest.raises(TypeError, match="qk_i8"):
        pkg.prefill_extend(**_call(), qk_i8="int8")


def test_bf16_pv_lane_is_refused_at_planning(pkg):
    with pytest.raises(pkg.CapabilityError, match=r"need_vb16=True") as info:
        pkg.plan_workspace(torch.device("cpu"), max_kv_len=64, max_q_len=8, need_vb16=True)
    assert info.value.field == "need_vb16"


def test_a_valid_request_passes_validation_and_only_then_reaches_the_device(pkg):
    with pytest.raises(RuntimeError, match=r"needs CUDA tensors"):
        pkg.prefill_extend(**_call())          # valid, but on the CPU: refused loudly, no fallback


def test_check_request_returns_the_derived_geometry(pkg):
    req = pkg.check_request(**_call())
    assert (req.q_len, req.q_heads, req.kv_heads, req.head_dim, req.kv_len, req.prefix) == (8, 24, 4, 256, 32, 24)
    assert req.sm_scale == 1.0 / 16.0 and req.kv_dtype == "bfloat16" and req.return_lse is False
    assert pkg.check_request(**_call(), sm_scale=0.25).sm_scale == 0.25


def test_int32_page_table_is_accepted(pkg):
    req = pkg.check_request(**_call(idx=torch.arange(KV_LEN, dtype=torch.int32)))
    assert req.kv_len == KV_LEN


def test_lse_and_supplied_buffers_are_accepted(pkg):
    call = _call()
    pkg.check_request(**call, return_lse=True,
                      out=torch.zeros_like(call["q"]),
                      lse_out=torch.zeros((Q_LEN, Q_HEADS), dtype=torch.float32))


def test_generalization_capability_widens_only_the_head_axes(pkg):
    gen = pkg.GENERALIZATION_CAPABILITY
    pkg.check_request(**_geometry(q_heads=8, kv_heads=2), capability=gen)
    with pytest.raises(pkg.CapabilityError, match=r"head_dim=128"):
        pkg.check_request(**_geometry(head_dim=128), capability=gen)
    with pytest.raises(pkg.CapabilityError, match=r"LSE output is not part of"):
        pkg.check_request(**_geometry(q_heads=8, kv_heads=2), capability=gen, return_lse=True)
    odd = pkg.OperatorCapability(operator_contract_version=1, layout_version=2, head_dim=(256,),
                                 q_heads=(6,), kv_heads=(4,), page_size=(1,), modes=("extend",),
                                 masks=("bottom_right_causal",))
    with pytest.raises(pkg.CapabilityError, match=r"q_heads=6 is not divisible by kv_heads=4"):
        pkg.check_supported(head_dim=256, q_heads=6, kv_heads=4, page_size=1, mode="extend",
                            mask="bottom_right_causal", kv_dtype="bfloat16", capability=odd)


def test_capability_surface_matches_the_contract(pkg):
    cap = pkg.V1_CAPABILITY
    assert cap.head_dim == (256,) and cap.q_heads == (16, 24, 32) and cap.kv_heads == (4,)
    assert cap.page_size == (1,) and cap.modes == ("extend",) and cap.masks == ("bottom_right_causal",)
    assert cap.kv_dtypes == ("bfloat16", "float16") and cap.returns_lse and cap.cuda_graph == "supported"
    for bad in (dict(page_size=16), dict(mode="decode"), dict(mask="causal")):
        args = dict(head_dim=256, q_heads=24, kv_heads=4, page_size=1, mode="extend",
                    mask="bottom_right_causal", kv_dtype="bfloat16")
        args.update(bad)
        with pytest.raises(pkg.CapabilityError):
            pkg.check_supported(**args)
