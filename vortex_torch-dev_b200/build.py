"""Build recipe for the C-ABI shared library (sm_100a only).

``python build.py`` compiles every ``csrc/*.cu`` with nvcc into ``lib/libvortex_b200.so``
next to this file.  nvcc cross-compiles, so no GPU is needed to build.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
CSRC = HERE / "csrc"
LIB_DIR = HERE / "lib"
LIB_PATH = LIB_DIR / "libvortex_b200.so"
# The same sources with -DVTX_CHECKED: every index a kernel reads and then uses as an address is compared with
# limits set through vtx_checked_set_limits.  Relocatable device code, because the limits live in one
# translation unit and are read from all of them.
CHECKED_LIB_PATH = LIB_DIR / "libvortex_b200_checked.so"
CHECKED_FLAGS = ["-DVTX_CHECKED", "-rdc=true"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the vortex_b200 library cannot be built")
    return cand


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def needs_build(checked: bool = False) -> bool:
    lib = CHECKED_LIB_PATH if checked else LIB_PATH
    if not lib.exists():
        return True
    t = lib.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list((ROOT / "include").glob("*.h"))
    return any(p.stat().st_mtime > t for p in deps)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False, checked: bool = False) -> Path:
    """Compile the library (``checked``: its checked twin) if it is missing or older than its sources; return its
    path."""
    lib = CHECKED_LIB_PATH if checked else LIB_PATH
    if not force and not needs_build(checked):
        return lib
    LIB_DIR.mkdir(exist_ok=True)
    objs = []
    obj_dir = HERE / ("build_checked" if checked else "build")
    obj_dir.mkdir(exist_ok=True)
    procs = []
    headers = list(CSRC.glob("*.cuh")) + list((ROOT / "include").glob("*.h"))
    newest_header = max((h.stat().st_mtime for h in headers), default=0.0)
    for src in sources():
        obj = obj_dir / (src.stem + ".o")
        objs.append(str(obj))
        # an object is reused when it is newer than its source and every header
        if (not force and not ptxas_info and obj.exists()
                and obj.stat().st_mtime > max(src.stat().st_mtime, newest_header)):
            continue
        cmd = [_nvcc(), *NVCC_FLAGS, *(CHECKED_FLAGS if checked else []), "-I", str(ROOT / "include"), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed on {src.name}:\n{out}\n")
        elif verbose or ptxas_info:
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("vortex_b200: compilation failed")
    tmp = lib.with_suffix(".so.tmp")
    cmd = [_nvcc(), "-shared", "-o", str(tmp), *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    if checked:
        cmd += ["-Xcompiler", "-fPIC"]  # the device-link step compiles a stub of its own
    subprocess.run(cmd, check=True)
    os.replace(tmp, lib)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv,
                checked="--checked" in sys.argv))
