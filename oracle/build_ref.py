"""Recipe for oracle/_ref/: the UNMODIFIED reference, installed for use as a checker and as the
same-box baseline.  Test infrastructure -- nothing in the product package imports it.

    python oracle/build_ref.py [--source /path/to/reference] [--no-ext]

1. `pip install --no-index --no-build-isolation --no-deps --target oracle/_ref <copy of the
   reference checkout>`: the reference's own Python package `attn_kernel_lab` (its CPU oracle
   `oracle_a.reference`, its preprocessing `quant`, its operator `ops.prefill_extend`).
2. Unless --no-ext: pre-builds the reference's own CUDA extension (its mma.sync kernel,
   src/attn_kernel_lab/csrc/fp8_prefill_attn.cu) for sm_100a with the flags its loader uses
   (src/attn_kernel_lab/kernel.py:186-196), into oracle/_ref/torch_ext, so that a GPU box
   loads it without a JIT build.  nvcc cross-compiles without a GPU.

oracle/_ref/ is listed in .gitignore (no reference source enters the history) and travels to
the GPU box with the working tree.  Where the reference checkout is absent (the GPU box), the
script does nothing and the prebuilt directory is used as it is.
"""
from __future__ import annotations

import argparse
import os
import pathlib
import shutil
import subprocess
import sys
import tempfile

HERE = pathlib.Path(__file__).resolve().parent
TARGET = HERE / "_ref"
EXT_DIR = TARGET / "torch_ext"
EXT_NAME = "attn_kernel_lab_fp8_prefill"          # the name the reference's loader uses


def install(source: pathlib.Path) -> None:
    with tempfile.TemporaryDirectory() as tmp:
        copy = pathlib.Path(tmp) / "reference"
        shutil.copytree(source, copy, ignore=shutil.ignore_patterns(".git", "__pycache__"))
        keep = EXT_DIR if EXT_DIR.exists() else None
        staged = None
        if keep is not None:                       # a rebuild of the Python side keeps the built extension
            staged = pathlib.Path(tmp) / "torch_ext"
            shutil.move(str(keep), str(staged))
        if TARGET.exists():
            shutil.rmtree(TARGET)
        subprocess.check_call([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation",
                               "--no-deps", "--quiet", "--find-links", "/opt/wheelhouse",
                               "--target", str(TARGET), str(copy)])
        if staged is not None:
            shutil.move(str(staged), str(EXT_DIR))


def build_extension() -> None:
    """The reference's extension for sm_100a, through the same tensor-library JIT call its own loader
    makes, into a build directory that travels."""
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ["TORCH_EXTENSIONS_DIR"] = str(EXT_DIR)
    EXT_DIR.mkdir(parents=True, exist_ok=True)
    sys.path.insert(0, str(TARGET))
    from attn_kernel_lab import kernel as ref_kernel
    from torch.utils.cpp_extension import load

    src = pathlib.Path(ref_kernel.__file__).resolve().parent / "csrc" / "fp8_prefill_attn.cu"
    load(name=EXT_NAME, sources=[str(src)], extra_cuda_cflags=["-O3", ref_kernel.gencode_for(10, 0)],
         verbose=False, is_python_module=False)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--source", default=os.environ.get("AKL_REFERENCE_SRC", "/root/reference"))
    ap.add_argument("--no-ext", action="store_true")
    args = ap.parse_args()
    source = pathlib.Path(args.source)
    if not (source / "src" / "attn_kernel_lab").is_dir():
        print(f"{source} is not a reference checkout: leaving {TARGET} as it is")
        return 0
    install(source)
    print(f"installed the reference package into {TARGET}")
    if not args.no_ext:
        build_extension()
        print(f"built the reference extension for sm_100a under {EXT_DIR}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
