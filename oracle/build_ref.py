"""Compile the reference's own greedy bit allocator, unmodified, into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  ``actnn/actnn/cpp_extension/calc_precision.cc`` of the reference
is host-only C++ (a torch/pybind11 extension with no CUDA in it), so it builds with ``g++``
straight from where it lies in the reference checkout; nothing is copied into this
repository and the output (``oracle/_ref/ref_calc_precision*.so``) is git-ignored.  The rest
of the reference's native code needs its CUDA build against an old PyTorch and is not
buildable here.

Usage:  python oracle/build_ref.py [path-to-reference-checkout]
The resulting module is loaded with :func:`load_ref_calc_precision`.
"""
from __future__ import annotations

import importlib.util
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
MOD_NAME = "ref_calc_precision"
DEFAULT_REFERENCE = os.environ.get("ACTNN_REFERENCE_ROOT")      # no built-in location: set it, or pass a path


def so_path() -> str:
    return os.path.join(OUT_DIR, MOD_NAME + ".so")


def build(reference_root: str = DEFAULT_REFERENCE, force: bool = False) -> str | None:
    """Build if the reference source is present; return the .so path (or None)."""
    out = so_path()
    if not reference_root:
        return out if os.path.exists(out) else None
    src = os.path.join(reference_root, "actnn", "actnn", "cpp_extension", "calc_precision.cc")
    if not os.path.exists(src):
        return out if os.path.exists(out) else None
    if os.path.exists(out) and not force and os.path.getmtime(out) >= os.path.getmtime(src):
        return out
    from torch.utils import cpp_extension
    import torch

    os.makedirs(OUT_DIR, exist_ok=True)
    inc = cpp_extension.include_paths() + [sysconfig.get_paths()["include"]]
    lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-DNDEBUG",
           "-DTORCH_EXTENSION_NAME=" + MOD_NAME, "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI))]
    cmd += ["-I" + p for p in inc]
    cmd += [src, "-o", out, "-L" + lib_dir, "-Wl,-rpath," + lib_dir,
            "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10"]
    subprocess.run(cmd, check=True)
    return out


def load_ref_calc_precision():
    """Import the built module (``.calc_precision(b, C, w, target)``); None if absent."""
    path = so_path()
    if not os.path.exists(path):
        return None
    import torch  # noqa: F401  (the extension links against libtorch)

    spec = importlib.util.spec_from_file_location(MOD_NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REFERENCE
    print(build(root, force=True))
