"""Build recipe for the optional reference cross-check extension (TEST INFRASTRUCTURE).

Compiles the reference project's own CUDA sources for its native decode-path functions
(``csrc/topk.cu``, ``csrc/utils_sglang.cu``, bound by ``csrc/register.cc``) where they lie in the
reference checkout, for sm_100, into ``oracle/_ref/vortex_torch_C_ref*.so``.  Nothing is copied into
this repository and the reference's own build system is not run: this is a direct nvcc/g++ compile
through ``torch.utils.cpp_extension`` with the output directory set to ``oracle/_ref``.

The GPU tests load the module (if it was built) to compare ``sglang_plan_decode`` and ``topk_output``
of the reference, bit for bit, with the sm_100a kernels of this repository on the same inputs.
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
MODULE = "vortex_torch_C_ref"
REFERENCE = Path(os.environ.get("VORTEX_REFERENCE_DIR", str(Path.home() / "reference")))
SOURCES = ["csrc/register.cc", "csrc/topk.cu", "csrc/utils_sglang.cu"]


def built_module_path():
    hits = sorted(OUT.glob(f"{MODULE}*.so")) if OUT.exists() else []
    return hits[0] if hits else None


def build(verbose: bool = False) -> Path:
    from torch.utils import cpp_extension

    srcs = [str(REFERENCE / s) for s in SOURCES]
    for s in srcs:
        if not os.path.isfile(s):
            raise FileNotFoundError(s)
    OUT.mkdir(exist_ok=True)
    build_dir = OUT / "build"
    build_dir.mkdir(exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    cpp_extension.load(
        name=MODULE,
        sources=srcs,
        extra_include_paths=[str(REFERENCE / "csrc")],
        extra_cflags=["-O2", f"-DTORCH_EXTENSION_NAME={MODULE}"],
        extra_cuda_cflags=["-O2", "-gencode", "arch=compute_100,code=sm_100"],
        build_directory=str(build_dir),
        is_python_module=False,  # just build the shared object; it is imported on the GPU box
        verbose=verbose,
    )
    so = build_dir / f"{MODULE}.so"
    dst = OUT / f"{MODULE}.so"
    shutil.copy2(so, dst)
    return dst


def build_if_possible() -> None:
    """Build when the reference checkout is present and the module is missing; never raises."""
    if built_module_path() is not None or not (REFERENCE / SOURCES[0]).is_file():
        return
    try:
        build()
    except Exception as exc:  # the cross-check is optional
        sys.stderr.write(f"oracle/build_ref: reference cross-check not built: {exc}\n")


def load():
    """Import the built module (GPU box).  Returns None when it was not built."""
    so = built_module_path()
    if so is None:
        return None
    import importlib.util

    import torch  # noqa: F401  (the extension links against libtorch)

    # the reference's binding file names its module "vortex_torch_C"; that fixes the init symbol
    spec = importlib.util.spec_from_file_location("vortex_torch_C", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(verbose=True))
