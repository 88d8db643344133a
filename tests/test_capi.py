"""The C-ABI boundary without a GPU: the library loads, exports every symbol include/akl.h
declares, agrees with the ctypes mirror on struct sizes, lays out workspaces sanely, and
rejects bad arguments on the host before any CUDA call."""
import ctypes
import pathlib
import re

import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]
HEADER = (ROOT / "include" / "akl.h").read_text()


@pytest.fixture(scope="module")
def K(pkg):
    from attn_kernel_lab_b200 import kernel

    return kernel


def declared_functions():
    body = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    return sorted(set(re.findall(r"\b(akl_[a-z0-9_]+)\s*\(", body)))


def test_library_exports_every_declared_symbol(K):
    lib = K.load()
    names = declared_functions()
    assert len(names) >= 13
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/akl.h but not exported"
    assert set(K.EXPORTS) <= set(names)
    assert lib.akl_abi_version() == int(re.search(r"#define AKL_ABI_VERSION (\d+)", HEADER).group(1))
    from attn_kernel_lab_b200 import kernel as K
    for name in ("AKL_FLAG_ROTATE", "AKL_FLAG_CENTER_K", "AKL_FLAG_QK_I8"):     # host constants == header
        assert getattr(K, name) == int(re.search(rf"#define {name} (\d+)u", HEADER).group(1)), name


def test_header_is_plain_c_with_reference_citations():
    code = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    assert 'extern "C"' in code and "torch" not in code and "#include <stdint.h>" in code
    assert code.count("#include") == 1                 # nothing but <stdint.h> crosses the boundary
    for cite in ("ops.py:485-609", ":253-336", "fp8_prefill_attn.cu:689-696"):
        assert cite in HEADER


def test_ctypes_mirror_matches_the_header_layout(K):
    assert ctypes.sizeof(K.Plan) == 16
    assert ctypes.sizeof(K.WsLayout) == 8 + 16 + 18 * 8
    # akl_call_t: 7 pointers + u64 + plan(16) + 13 x 4-byte scalars, padded to 8
    assert ctypes.sizeof(K.Call) == 7 * 8 + 8 + 16 + 13 * 4 + 4
    assert ctypes.sizeof(K.Merge) == 4 * 8 + 8
    assert K.Call.sm_scale.offset == K.Call.flags.offset + 4


def test_error_strings(K):
    lib = K.load()
    for code in (0, -1, -2, -3, -4, -5, -6):
        assert lib.akl_strerror(code)
    assert b"unknown" in lib.akl_strerror(-99)
    with pytest.raises(K.NativeError) as info:
        K.check(K.AKL_ERR_CAPACITY, "here")
    assert info.value.code == K.AKL_ERR_CAPACITY and "here" in str(info.value)


def test_workspace_layout_arithmetic(K):
    L = K.workspace_layout(10240, 2048, 24, 4)
    assert (L.npairs, L.ntiles, L.mtiles) == (80, 160, 16)
    offs = [getattr(L, f[0]) for f in K.WsLayout._fields_ if f[0].startswith("off_")]
    assert offs == sorted(offs) and all(o % 1024 == 0 for o in offs) and L.total_bytes > offs[-1]
    assert L.off_qscale - L.off_q8 == 24 * 16 * 32768
    assert L.off_v8t - L.off_k8 == 4 * 80 * 32768
    # ragged maxima round up to whole tiles
    L2 = K.workspace_layout(65, 5, 16, 4)
    assert (L2.npairs, L2.ntiles, L2.mtiles) == (1, 2, 1)
    lib = K.load()
    out = K.WsLayout()
    assert lib.akl_workspace_layout(ctypes.byref(K.Plan(0, 8, 24, 4)), ctypes.byref(out)) == K.AKL_ERR_INVALID
    assert lib.akl_workspace_layout(ctypes.byref(K.Plan(8, 8, 24, 5)), ctypes.byref(out)) == K.AKL_ERR_UNSUPPORTED
    assert lib.akl_workspace_layout(None, ctypes.byref(out)) == K.AKL_ERR_INVALID


def _host_call(K, **over):
    """A call whose pointers are never dereferenced: every case below fails host validation."""
    L = K.workspace_layout(256, 128, 24, 4)
    c = K.Call()
    c.q = c.k_pool = c.v_pool = c.idx = c.out = 4096
    c.workspace = 1 << 20
    c.workspace_bytes = int(L.total_bytes)
    c.plan = K.Plan(256, 128, 24, 4)
    c.T, c.N, c.prefix, c.q_heads, c.kv_heads = 64, 256, 192, 24, 4
    c.sm_scale = 0.0625
    for k, v in over.items():
        setattr(c, k, v)
    return c


@pytest.mark.parametrize("over,code", [
    (dict(T=0), -1), (dict(N=0), -1), (dict(prefix=-1), -1), (dict(kv_dtype=7), -1),
    (dict(idx_dtype=3), -1), (dict(sm_scale=0.0), -1), (dict(kv_pos0=32), -1),
    (dict(workspace=None), -1), (dict(idx=None), -1),
    (dict(q_heads=25), -2),
    (dict(N=257), -3), (dict(T=129), -3), (dict(workspace_bytes=1024), -3), (dict(q_heads=16), -3),
    (dict(workspace=(1 << 20) + 16), -5), (dict(q=4104), -5),
    (dict(prefix=193), -1),          # prefix > N - T
    (dict(kv_pos0=64), -1),          # a split request must use the phase entry points
], ids=lambda v: str(v))
def test_host_side_argument_checks_run_before_any_cuda_call(K, over, code):
    lib = K.load()
    c = _host_call(K, **over)
    assert lib.akl_prefill_extend(ctypes.byref(c), None) == code
    assert lib.akl_prefill_extend(None, None) == K.AKL_ERR_INVALID


def test_merge_argument_checks(K):
    lib = K.load()
    assert lib.akl_merge_states(None, None) == K.AKL_ERR_INVALID
    m = K.Merge(4096, 4096, 4096, None, 0, 16)
    assert lib.akl_merge_states(ctypes.byref(m), None) == K.AKL_ERR_INVALID
    m = K.Merge(4096, 4096, 4096, None, 65, 16)
    assert lib.akl_merge_states(ctypes.byref(m), None) == K.AKL_ERR_INVALID


def test_loader_fails_loudly_when_the_library_is_missing(K, monkeypatch, tmp_path):
    monkeypatch.setattr(K, "_lib", None)
    monkeypatch.setattr(K, "LIB_PATH", tmp_path / "libakl_sm100a.so")
    with pytest.raises(RuntimeError, match=r"no CPU or tensor-library fallback"):
        K.load()


def test_build_uses_the_arch_specific_target(K):
    assert K.GENCODE == "arch=compute_100a,code=sm_100a"
    assert K.EXTRA_FLAGS["akl_prep.cu"] == ("-fmad=false",)
    assert len(K.source_build_id()) == 16


# ------------------------------------------------------------------ workspace semantics (host)
def test_capacity_workspace_never_moves_and_refuses_to_grow(pkg):
    cpu = torch.device("cpu")
    ws = pkg.plan_workspace(cpu, max_kv_len=1000, max_q_len=200, q_heads=24, kv_heads=4)
    plan = ws.capacity
    assert (plan.npad, plan.ntmax, plan.mpad) == (1024, 16, 256) and plan.admits(1000, 200) and not plan.admits(1001, 1)
    before = ws.buffer_pointers()
    assert before["q8"] % 1024 == 0 and len(before) == 18
    ws.ensure(1000, 200, 24, 4)
    ws.ensure(1, 1, 24, 4)
    assert ws.buffer_pointers() == before
    for bad in ((1001, 200, 24, 4), (1000, 201, 24, 4), (1000, 200, 32, 4)):
        with pytest.raises(pkg.WorkspaceCapacityError, match=r"outside the capacity plan"):
            ws.ensure(*bad)
    assert not issubclass(pkg.WorkspaceCapacityError, pkg.CapabilityError)
    ws.release_capacity()
    ws.ensure(2000, 200, 24, 4)
    assert ws.capacity is None and ws.dims[0] == 2000


def test_growing_workspace_keeps_earlier_phase_results(pkg):
    ws = pkg.FP8PrefillWorkspace(torch.device("cpu"))
    ws.ensure(300, 10, 16, 4)
    ws.view("kscale").fill_(3.0)
    ws.view("k8")[:, :, :, :, :] = 7
    ws.ensure(300, 500, 16, 4)                       # the q side grows
    assert ws.dims == (300, 500, 16, 4)
    assert bool((ws.view("kscale") == 3.0).all()) and bool((ws.view("k8") == 7).all())
    with pytest.raises(ValueError, match=r"BOTH max_kv_len and max_q_len"):
        pkg.FP8PrefillWorkspace(torch.device("cpu"), max_kv_len=10)
    with pytest.raises(ValueError, match=r"must be an int >= 1"):
        ws.reserve(0, 5)
    with pytest.raises(ValueError, match=r"divisible"):
        ws.reserve(5, 5, q_heads=10, kv_heads=4)


def test_logical_views_undo_the_swizzle(pkg):
    """q8/k8/v8 logical views are the inverse of the tile-image addressing the kernels use:
    byte (row r, column c) of a [128][128 B] plane lives at r*128 + ((c/16 ^ r%8)*16 + c%16)."""
    ws = pkg.FP8PrefillWorkspace(torch.device("cpu"), max_kv_len=200, max_q_len=130, q_heads=16, kv_heads=4)
    q8 = ws.view("q8")
    q8.zero_()
    h, row, col = 3, 129, 200                         # tile 1, row 1, plane 1, byte 72
    r, c = row % 128, col % 128
    q8[h, row // 128, col // 128].view(-1)[r * 128 + ((((c >> 4) ^ (r & 7)) << 4) | (c & 15))] = 0x5A
    logical = ws.q8_logical(130)
    assert logical.shape == (16, 256, 256) and int(logical[h, row, col]) == 0x5A and int(logical.sum()) == 0x5A
    v8t = ws.view("v8t")
    v8t.zero_()
    kvh, key, d = 2, 150, 77                          # pair 1, key 22 inside the pair
    kk = key % 128
    v8t[kvh, key // 128].view(-1)[d * 128 + ((((kk >> 4) ^ (d & 7)) << 4) | (kk & 15))] = 0x33
    vlog = ws.v8_logical(200)
    assert vlog.shape == (4, 256, 256) and int(vlog[kvh, key, d]) == 0x33 and int(vlog.sum()) == 0x33


# ------------------------------------------------------------------ argument validation, host side only
def _fake_call(K, **over):
    """A call that would be valid if its pointers were real.  Every test below changes one field so
    that validation refuses the call before anything is launched or dereferenced."""
    lib = K.load()
    plan = K.Plan(4096, 256, 24, 4)
    lay = K.WsLayout()
    assert lib.akl_workspace_layout(ctypes.byref(plan), ctypes.byref(lay)) == K.AKL_OK
    c = K.Call()
    c.q, c.k_pool, c.v_pool, c.idx, c.out = 0x10000, 0x20000, 0x30000, 0x40000, 0x50000
    c.lse_out = None
    c.workspace, c.workspace_bytes, c.plan = 0x100000, lay.total_bytes, plan
    c.T, c.N, c.prefix, c.q_heads, c.kv_heads = 64, 320, 256, 24, 4
    c.kv_dtype, c.idx_dtype = K.AKL_KV_BF16, K.AKL_IDX_I64
    c.flags, c.sm_scale = K.AKL_FLAG_ROTATE | K.AKL_FLAG_CENTER_K, 1.0 / 16.0
    c.kv_pos0 = c.n_total = c.tile0_global = c.ntiles_global = 0
    for k, v in over.items():
        setattr(c, k, v)
    return lib, c


@pytest.mark.parametrize("field, value, code", [
    ("T", 0, "AKL_ERR_INVALID"),
    ("N", 0, "AKL_ERR_INVALID"),
    ("prefix", -1, "AKL_ERR_INVALID"),
    ("kv_dtype", 7, "AKL_ERR_INVALID"),
    ("idx_dtype", 5, "AKL_ERR_INVALID"),
    ("sm_scale", 0.0, "AKL_ERR_INVALID"),
    ("kv_pos0", 32, "AKL_ERR_INVALID"),              # a split starts on a 64-key tile boundary
    ("flags", 8, "AKL_ERR_INVALID"),                 # unknown mode bit
    ("workspace", None, "AKL_ERR_INVALID"),
    ("kv_heads", 5, "AKL_ERR_UNSUPPORTED"),          # 24 q heads do not divide over 5
    ("q_heads", 32, "AKL_ERR_CAPACITY"),             # not the head count the workspace was planned for
    ("workspace_bytes", 4096, "AKL_ERR_CAPACITY"),
    ("N", 4097, "AKL_ERR_CAPACITY"),                 # one key more than the plan's maximum tiles hold
    ("T", 257, "AKL_ERR_CAPACITY"),
    ("k_pool", 0x20008, "AKL_ERR_ALIGN"),
    ("out", 0x50004, "AKL_ERR_ALIGN"),
    ("workspace", 0x100200, "AKL_ERR_ALIGN"),        # 16-byte but not 1024-byte aligned
    ("tile0_global", -1, "AKL_ERR_INVALID"),         # would index the tile-sum arrays before their start
    ("tile0_global", 2, "AKL_ERR_INVALID"),          # disagrees with kv_pos0 = 0
    ("ntiles_global", -3, "AKL_ERR_INVALID"),
    ("n_total", -5, "AKL_ERR_INVALID"),
    ("n_total", 319, "AKL_ERR_INVALID"),             # global length shorter than this call's positions
])
def test_native_entry_refuses_bad_arguments_before_any_launch(K, field, value, code):
    lib, c = _fake_call(K, **{field: value})
    for fn in ("akl_prefill_extend", "akl_kv_tile_stats", "akl_kv_transform", "akl_attention"):
        assert getattr(lib, fn)(ctypes.byref(c), None) == getattr(K, code), (fn, field)
    assert lib.akl_strerror(getattr(K, code)).decode()


@pytest.mark.parametrize("over, code", [
    (dict(kv_pos0=64, tile0_global=1, n_total=0, ntiles_global=6), "AKL_ERR_INVALID"),  # split without a global length
    (dict(kv_pos0=64, tile0_global=0x7FFFFFF0, n_total=384, ntiles_global=6), "AKL_ERR_INVALID"),  # int overflow bait
    (dict(kv_pos0=64, tile0_global=1, n_total=384, ntiles_global=5), "AKL_ERR_INVALID"),  # written tiles beyond the global range
    (dict(kv_pos0=64, tile0_global=1, n_total=383, ntiles_global=6), "AKL_ERR_INVALID"),  # divisor smaller than kv_pos0 + N
    (dict(kv_pos0=64, tile0_global=1, n_total=8192, ntiles_global=128), "AKL_ERR_CAPACITY"),  # more global tiles than the plan
])
def test_kv_split_fields_are_checked_together_on_the_host(K, over, code):
    """The phase entry points take the KV-axis split fields; an inconsistent combination must be
    refused before any launch (a negative or overflowing tile index would be an out-of-bounds
    device store).  The consistent combinations run in the GPU split tests."""
    lib, c = _fake_call(K, **over)
    for fn in ("akl_kv_tile_stats", "akl_kv_means", "akl_kv_scales", "akl_kv_transform", "akl_attention"):
        assert getattr(lib, fn)(ctypes.byref(c), None) == getattr(K, code), (fn, over)
