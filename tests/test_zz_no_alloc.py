"""The allocation-free entry point, `akl_prefill_extend_static_scratch`.

Who needs it: a host that cannot allocate device memory where it calls the operator -- a plugin
inside an engine that owns all memory and lends none, or a process whose pool is frozen after
start-up.  The library then works out of a 16 MiB array of its own instead of a caller-provided
workspace.  It must give exactly what `akl_prefill_extend` gives (same kernels, same arithmetic:
bit-equal BF16 output and base-2 LSE), on consecutive calls that reuse the array with different
data, and it must refuse what does not fit.  Collected last on purpose: a run that stops at the
first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

import cases
import helpers

pytestmark = pytest.mark.gpu


def _run_both(pkg, cuda, case):
    from attn_kernel_lab_b200 import kernel as K, quant

    lib = K.load()
    inp = cases.make_inputs(case)
    q, kp, vp, idx = (inp[k].to(cuda) for k in ("q", "k_pool", "v_pool", "idx"))
    T, H, N, KVH = case["T"], case["H"], case["N"], case["KVH"]
    ref_out, ref_lse = helpers.fp8_extend(pkg, q, kp, vp, idx, case["prefix"], sm_scale=case["sm_scale"],
                                          rotate=case["rotate"], center_k=case["center_k"], return_lse=True)
    out = torch.full_like(q, float("nan"))
    lse = torch.full((T, H), float("nan"), dtype=torch.float32, device=cuda)
    holder = quant.FP8PrefillWorkspace(cuda, max_kv_len=64, max_q_len=1, q_heads=H, kv_heads=KVH)
    call = quant.make_call(holder, q=q, k_pool=kp, v_pool=vp, idx=idx, out=out, lse_out=lse, q_len=T,
                           kv_len=N, prefix=case["prefix"], q_heads=H, kv_heads=KVH,
                           sm_scale=case["sm_scale"], rotate=case["rotate"], center_k=case["center_k"])
    call.workspace = None            # the entry point must not look at the caller's workspace fields
    call.workspace_bytes = 0
    before = torch.cuda.memory_allocated(cuda)
    code = lib.akl_prefill_extend_static_scratch(ctypes.byref(call), torch.cuda.current_stream().cuda_stream)
    K.check(code, "akl_prefill_extend_static_scratch")
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(cuda) == before
    return (ref_out, ref_lse), (out, lse)


def test_static_scratch_entry_point_equals_the_workspace_entry_point_twice_in_a_row(pkg, cuda):
    first = cases.GOLDEN_CASES[0]                                  # 256 cached + 64 new, 24:4
    second = cases._case("zz_second", 200, 1500, 1300, 32, 4, "scattered", "jitter", 9901,
                         kv_dtype="float16")                       # larger, other heads, other dtype
    for case in (first, second, first):
        (ref_out, ref_lse), (out, lse) = _run_both(pkg, cuda, case)
        assert torch.equal(out, ref_out), case["name"]
        assert torch.equal(lse, ref_lse), case["name"]


def test_static_scratch_entry_point_refuses_what_does_not_fit(pkg, cuda):
    from attn_kernel_lab_b200 import kernel as K, quant

    lib = K.load()
    n, t, h = 8192, 256, 24                                        # layout needs 19.5 MiB > 16 MiB
    q = torch.zeros((t, h, 256), dtype=torch.bfloat16, device=cuda)
    pool = torch.zeros((n, 4, 256), dtype=torch.bfloat16, device=cuda)
    idx = torch.arange(n, device=cuda)
    holder = quant.FP8PrefillWorkspace(cuda, max_kv_len=64, max_q_len=1, q_heads=h, kv_heads=4)
    call = quant.make_call(holder, q=q, k_pool=pool, v_pool=pool, idx=idx, out=torch.empty_like(q), q_len=t,
                           kv_len=n, prefix=n - t, q_heads=h, kv_heads=4, sm_scale=0.0625)
    code = lib.akl_prefill_extend_static_scratch(ctypes.byref(call), torch.cuda.current_stream().cuda_stream)
    assert code == K.AKL_ERR_CAPACITY
    with pytest.raises(K.NativeError, match="does not fit"):
        K.check(code, "akl_prefill_extend_static_scratch")
    assert lib.akl_prefill_extend_static_scratch(None, None) == K.AKL_ERR_INVALID


def test_static_scratch_status_is_observable_and_a_refused_call_enqueues_nothing(pkg, cuda):
    """The status word of this entry point lives inside the library's own array, so the library
    hands it out itself; and a call refused on the host (here: a prefix out of range) must not
    clear the status an earlier call left, nor enqueue anything."""
    from attn_kernel_lab_b200 import kernel as K

    lib = K.load()
    case = cases.GOLDEN_CASES[0]
    _run_both(pkg, cuda, case)
    host = torch.full((1,), 77, dtype=torch.int32).pin_memory()
    st = torch.cuda.current_stream().cuda_stream
    K.check(lib.akl_static_scratch_status(host.data_ptr(), st), "akl_static_scratch_status")
    torch.cuda.synchronize()
    assert int(host[0]) == 0, "a clean call leaves status 0"
    assert lib.akl_static_scratch_status(None, st) == K.AKL_ERR_INVALID

    from attn_kernel_lab_b200 import quant

    inp = cases.make_inputs(case)
    q, kp, vp, idx = (inp[k].to(cuda) for k in ("q", "k_pool", "v_pool", "idx"))
    holder = quant.FP8PrefillWorkspace(cuda, max_kv_len=64, max_q_len=1, q_heads=case["H"], kv_heads=case["KVH"])
    out = torch.full_like(q, 3.0)
    call = quant.make_call(holder, q=q, k_pool=kp, v_pool=vp, idx=idx, out=out, q_len=case["T"], kv_len=case["N"],
                           prefix=case["N"], q_heads=case["H"], kv_heads=case["KVH"], sm_scale=case["sm_scale"])
    assert lib.akl_prefill_extend_static_scratch(ctypes.byref(call), st) == K.AKL_ERR_INVALID
    torch.cuda.synchronize()
    assert bool((out == 3.0).all()), "nothing ran"
