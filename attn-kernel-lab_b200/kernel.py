"""Build and load libakl_sm100a.so, the C-ABI library behind the operator.

Takes the place of the reference's wheel-or-JIT loader of a pybind11 torch extension
(src/attn_kernel_lab/kernel.py:151-196).  There is no tensor-library header in the native
code, so the build is a handful of plain `nvcc -c` runs plus a link, and the binding is `ctypes`
over the structs of include/akl.h.

There is no fallback: `load()` raises if the library is missing or lacks a symbol.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import pathlib
import shutil
import subprocess
import threading
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = pathlib.Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
LIB_NAME = "libakl_sm100a.so"
LIB_PATH = PKG_DIR / LIB_NAME

#: Explicit -gencode, never a bare -arch: tcgen05 needs the arch-specific target.
GENCODE = "arch=compute_100a,code=sm_100a"
SOURCES = ("akl_prep.cu", "akl_attn_sm100.cu", "akl_merge.cu", "akl_api.cu", "akl_static_scratch.cu")
#: Per-file extra flags.  The preprocessing kernels decide quantised bytes, so no
#: multiply-add may be contracted there.
EXTRA_FLAGS = {"akl_prep.cu": ("-fmad=false",)}

EXPORTS = (
    "akl_abi_version", "akl_strerror", "akl_last_cuda_error", "akl_workspace_layout",
    "akl_prefill_extend", "akl_kv_tile_stats", "akl_kv_means", "akl_kv_scales",
    "akl_kv_transform", "akl_quantize_q", "akl_attention", "akl_attention_dump",
    "akl_merge_states", "akl_prefill_extend_static_scratch",
    "akl_batch_layout", "akl_batch_plan", "akl_prefill_extend_batch", "akl_prefill_extend_batch_phases",
    "akl_selftest_exact_division", "akl_static_scratch_status",
)

AKL_OK = 0
AKL_ERR_INVALID, AKL_ERR_UNSUPPORTED, AKL_ERR_CAPACITY = -1, -2, -3
AKL_ERR_CUDA, AKL_ERR_ALIGN, AKL_ERR_TIMEOUT = -4, -5, -6
AKL_KV_BF16, AKL_KV_FP16 = 0, 1
AKL_IDX_I64, AKL_IDX_I32 = 0, 1
AKL_FLAG_ROTATE, AKL_FLAG_CENTER_K, AKL_FLAG_QK_I8 = 1, 2, 4
AKL_BATCH_STATS, AKL_BATCH_MEANS, AKL_BATCH_TRANSFORM, AKL_BATCH_ATTENTION, AKL_BATCH_ALL = 1, 2, 4, 8, 15


class Plan(ctypes.Structure):
    _fields_ = [("max_kv_len", ctypes.c_int32), ("max_q_len", ctypes.c_int32),
                ("q_heads", ctypes.c_int32), ("kv_heads", ctypes.c_int32)]


class WsLayout(ctypes.Structure):
    _fields_ = [("total_bytes", ctypes.c_uint64),
                ("npairs", ctypes.c_int32), ("ntiles", ctypes.c_int32),
                ("mtiles", ctypes.c_int32), ("reserved_", ctypes.c_int32)] + [
        (name, ctypes.c_uint64) for name in (
            "off_q8", "off_qscale", "off_k8", "off_v8t", "off_kscale", "off_vst", "off_vlog2r",
            "off_vinvr", "off_vam", "off_vscale", "off_vsmax", "off_kmean", "off_vmean",
            "off_ktsum", "off_vtsum", "off_vtmax", "off_vtmin", "off_status")]


class Call(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p), ("k_pool", ctypes.c_void_p), ("v_pool", ctypes.c_void_p),
        ("idx", ctypes.c_void_p), ("out", ctypes.c_void_p), ("lse_out", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_uint64),
        ("plan", Plan),
        ("T", ctypes.c_int32), ("N", ctypes.c_int32), ("prefix", ctypes.c_int32),
        ("q_heads", ctypes.c_int32), ("kv_heads", ctypes.c_int32),
        ("kv_dtype", ctypes.c_int32), ("idx_dtype", ctypes.c_int32),
        ("flags", ctypes.c_uint32), ("sm_scale", ctypes.c_float),
        ("kv_pos0", ctypes.c_int32), ("n_total", ctypes.c_int32),
        ("tile0_global", ctypes.c_int32), ("ntiles_global", ctypes.c_int32),
    ]


class Merge(ctypes.Structure):
    _fields_ = [("parts_o", ctypes.c_void_p), ("parts_lse", ctypes.c_void_p),
                ("out", ctypes.c_void_p), ("lse_out", ctypes.c_void_p),
                ("nparts", ctypes.c_int32), ("rows", ctypes.c_int32)]


class BatchCaps(ctypes.Structure):
    _fields_ = [("max_requests", ctypes.c_int32), ("max_total_kv_pairs", ctypes.c_int32),
                ("max_total_q_tiles", ctypes.c_int32), ("q_heads", ctypes.c_int32),
                ("kv_heads", ctypes.c_int32), ("reserved_", ctypes.c_int32)]


class BatchLayout(ctypes.Structure):
    _fields_ = [("workspace_bytes", ctypes.c_uint64), ("table_bytes", ctypes.c_uint64),
                ("ws_off_status", ctypes.c_uint64),
                ("table_off_geoms", ctypes.c_uint32), ("table_geom_stride", ctypes.c_uint32),
                ("table_off_stat_totals", ctypes.c_uint32), ("table_off_qcta_totals", ctypes.c_uint32),
                ("table_off_items", ctypes.c_uint32), ("reserved_", ctypes.c_uint32)]


class BatchRequest(ctypes.Structure):
    _fields_ = [("q", ctypes.c_void_p), ("k_pool", ctypes.c_void_p), ("v_pool", ctypes.c_void_p),
                ("idx", ctypes.c_void_p), ("out", ctypes.c_void_p), ("lse_out", ctypes.c_void_p),
                ("T", ctypes.c_int32), ("N", ctypes.c_int32), ("prefix", ctypes.c_int32),
                ("reserved_", ctypes.c_int32)]


class Batch(ctypes.Structure):
    _fields_ = [("caps", BatchCaps), ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_uint64),
                ("table", ctypes.c_void_p), ("table_bytes", ctypes.c_uint64),
                ("kv_dtype", ctypes.c_int32), ("idx_dtype", ctypes.c_int32),
                ("flags", ctypes.c_uint32), ("sm_scale", ctypes.c_float)]


class NativeError(RuntimeError):
    """A native entry point returned a code other than AKL_OK (a defect or a CUDA failure,
    never an out-of-surface request: those are rejected in Python before any native call)."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


def source_build_id() -> str:
    """sha256 over the native sources and the public header (the reference keys its build on
    a source hash the same way, kernel.py:65-81)."""
    h = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [INCLUDE / "akl.h"]):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    return h.hexdigest()[:16]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libakl_sm100a.so cannot be built")
    return exe


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    """Compile every .cu for sm_100a and link libakl_sm100a.so next to this file."""
    stamp = PKG_DIR / "build" / "build_id"
    build_id = source_build_id()
    if not force and LIB_PATH.exists() and stamp.exists() and stamp.read_text() == build_id:
        return LIB_PATH
    objdir = PKG_DIR / "build"
    objdir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    sources = list(SOURCES)
    common = [nvcc, "-gencode", GENCODE, "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v", f"-I{INCLUDE}"]

    def compile_one(src: str):
        obj = objdir / (src[:-3] + ".o")
        cmd = common + list(EXTRA_FLAGS.get(src, ())) + ["-c", str(CSRC / src), "-o", str(obj)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        (objdir / (src[:-3] + ".ptxas.log")).write_text(proc.stderr)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{proc.stderr}")
        if verbose:
            print(proc.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=len(sources)) as pool:
        objs = list(pool.map(compile_one, sources))
    link = [nvcc, "-shared", "-gencode", GENCODE, "-o", str(LIB_PATH)] + [str(o) for o in objs]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed:\n{proc.stderr}")
    stamp.write_text(build_id)
    return LIB_PATH


_lib = None
_lock = threading.Lock()


def load():
    """The loaded library with argument types set.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -c \"import attn_kernel_lab_b200 as a; "
                "a.build()\"` (needs nvcc).  This operator has no CPU or tensor-library fallback."
            )
        lib = ctypes.CDLL(str(LIB_PATH))
        missing = [name for name in EXPORTS if not hasattr(lib, name)]
        if missing:
            raise RuntimeError(f"{LIB_PATH} lacks symbols {missing}: rebuild it")
        lib.akl_abi_version.restype = ctypes.c_int
        lib.akl_strerror.restype = ctypes.c_char_p
        lib.akl_strerror.argtypes = [ctypes.c_int]
        lib.akl_last_cuda_error.restype = ctypes.c_char_p
        lib.akl_workspace_layout.argtypes = [ctypes.POINTER(Plan), ctypes.POINTER(WsLayout)]
        for name in ("akl_prefill_extend", "akl_prefill_extend_static_scratch", "akl_kv_tile_stats", "akl_kv_means", "akl_kv_scales",
                     "akl_kv_transform", "akl_quantize_q", "akl_attention"):
            fn = getattr(lib, name)
            fn.argtypes = [ctypes.POINTER(Call), ctypes.c_void_p]
            fn.restype = ctypes.c_int
        lib.akl_attention_dump.argtypes = [ctypes.POINTER(Call), ctypes.c_void_p, ctypes.c_void_p,
                                           ctypes.c_void_p]
        lib.akl_attention_dump.restype = ctypes.c_int
        lib.akl_merge_states.argtypes = [ctypes.POINTER(Merge), ctypes.c_void_p]
        lib.akl_merge_states.restype = ctypes.c_int
        lib.akl_batch_layout.argtypes = [ctypes.POINTER(BatchCaps), ctypes.POINTER(BatchLayout)]
        lib.akl_batch_layout.restype = ctypes.c_int
        lib.akl_batch_plan.argtypes = [ctypes.POINTER(Batch), ctypes.POINTER(BatchRequest), ctypes.c_int32,
                                       ctypes.c_void_p]
        lib.akl_batch_plan.restype = ctypes.c_int
        lib.akl_prefill_extend_batch.argtypes = [ctypes.POINTER(Batch), ctypes.c_void_p]
        lib.akl_prefill_extend_batch.restype = ctypes.c_int
        lib.akl_prefill_extend_batch_phases.argtypes = [ctypes.POINTER(Batch), ctypes.c_uint32, ctypes.c_void_p]
        lib.akl_prefill_extend_batch_phases.restype = ctypes.c_int
        lib.akl_selftest_exact_division.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
        lib.akl_selftest_exact_division.restype = ctypes.c_int
        lib.akl_static_scratch_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        lib.akl_static_scratch_status.restype = ctypes.c_int
        _lib = lib
    return _lib


def check(code: int, where: str) -> None:
    """Turn a native return code into an exception."""
    if code == AKL_OK:
        return
    lib = load()
    msg = lib.akl_strerror(code).decode()
    if code == AKL_ERR_CUDA:
        msg += ": " + lib.akl_last_cuda_error().decode()
    raise NativeError(code, f"{where}: {msg} (code {code})")


def workspace_layout(max_kv_len: int, max_q_len: int, q_heads: int, kv_heads: int) -> WsLayout:
    lib = load()
    plan = Plan(max_kv_len, max_q_len, q_heads, kv_heads)
    out = WsLayout()
    check(lib.akl_workspace_layout(ctypes.byref(plan), ctypes.byref(out)), "akl_workspace_layout")
    return out
