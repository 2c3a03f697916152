"""In-tree build of the native extension ``torchcomms_b200/_comms.so``.

Every ``.cpp`` / ``.cu`` under ``csrc/`` goes into one shared object compiled
for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``).  The build uses
``torch.utils.cpp_extension.load`` (ninja, incremental) with its work files
under ``build/`` and copies the result next to this file, so importing the
package never triggers a compile.  nvcc cross-compiles without a GPU.

Run ``python -m torchcomms_b200._build`` (add ``-v`` for the compiler lines).
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR.parent / "build" / "comms_ext"
TARGET = PKG_DIR / "_comms.so"

CUDA_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xptxas",
    "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fvisibility=hidden", "-Wno-unused-variable"]


def sources() -> list[str]:
    out = []
    for pattern in ("**/*.cpp", "**/*.cu"):
        out.extend(str(p) for p in sorted(CSRC.glob(pattern)))
    return out


def needs_build() -> bool:
    if not TARGET.exists():
        return True
    newest = max(
        p.stat().st_mtime
        for pattern in ("**/*.cpp", "**/*.cu", "**/*.hpp", "**/*.cuh", "**/*.h")
        for p in CSRC.glob(pattern)
    )
    return newest > TARGET.stat().st_mtime


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile (if sources changed) and return the path of the shared object."""
    if not force and not needs_build():
        return TARGET
    from torch.utils import cpp_extension

    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    # The extension must share the process's libstdc++.so.6 with PyTorch. A
    # toolchain whose libstdc++.so link is broken silently falls back to the
    # static archive, and two copies of the locale/iostream state in one
    # process crash on the first formatted number. Prefer the system driver
    # and verify the result below.
    for var, exe in (("CXX", "/usr/bin/g++"), ("CC", "/usr/bin/gcc")):
        override = os.environ.get("B200COMMS_" + var)
        if override:
            os.environ[var] = override
        elif os.path.exists(exe):
            os.environ[var] = exe
    cpp_extension.load(
        name="_comms",
        sources=sources(),
        extra_cflags=CXX_FLAGS,
        extra_cuda_cflags=CUDA_FLAGS,
        extra_ldflags=["-ldl", "-lpthread"],
        extra_include_paths=[str(CSRC)],
        build_directory=str(BUILD_DIR),
        with_cuda=True,
        is_python_module=False,
        verbose=verbose,
    )
    built = BUILD_DIR / "_comms.so"
    if not built.exists():
        raise RuntimeError(f"build finished but {built} is missing")
    import subprocess

    needed = subprocess.run(["ldd", str(built)], capture_output=True, text=True).stdout
    if "libstdc++.so" not in needed:
        raise RuntimeError(
            f"{built} does not link libstdc++.so dynamically; set B200COMMS_CXX to a g++ "
            "whose libstdc++.so resolves"
        )
    tmp = TARGET.with_suffix(".so.tmp")
    shutil.copy2(built, tmp)
    os.replace(tmp, TARGET)
    return TARGET


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(path)
