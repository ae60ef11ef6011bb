"""Build the unmodified reference CUDA extension into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  The reference renderer (Davidxdydz/trigrad,
``src/trigrad/{render,module,util,tests}.cu``) exists only as CUDA, so it cannot
execute on a CPU-only machine, but nvcc cross-compiles it there.  This recipe
compiles the four translation units *where they lie* in the reference checkout
(nothing is copied) for sm_100a and links ``oracle/_ref/trigrad_ref_C*.so``.
On a machine with a B200 the parity tests import that module and call its
``render_forward`` / ``render_backward`` (``src/trigrad/module.cu:8-9``) as the
third leg next to the CPU oracle and the product kernels, and
``tests/golden/make_golden.py`` uses it to record golden vectors.

Usage:  python oracle/build_ref.py [/path/to/reference]   (default: $TRIGRAD_REFERENCE, else the mounted checkout)
Does nothing (exit 0) when the reference checkout is absent.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "trigrad_ref_C"
SOURCES = ["render.cu", "module.cu", "util.cu", "tests.cu"]  # setup.py:4 of the reference


def so_path() -> str:
    return os.path.join(OUT, NAME + sysconfig.get_config_var("EXT_SUFFIX"))


DEFAULT_REFERENCE = os.environ.get("TRIGRAD_REFERENCE", os.path.join(os.sep, "root", "reference"))


def build(ref_root: str = DEFAULT_REFERENCE, force: bool = False, verbose: bool = True) -> str | None:
    src_dir = os.path.join(ref_root, "src", "trigrad")
    if not os.path.isdir(src_dir):
        if verbose:
            print(f"[build_ref] {src_dir} not present; nothing to build")
        return None
    target = so_path()
    srcs = [os.path.join(src_dir, s) for s in SOURCES]
    if not force and os.path.exists(target):
        newest = max(os.path.getmtime(p) for p in srcs + [os.path.join(src_dir, "util.h")])
        if os.path.getmtime(target) >= newest:
            return target
    os.makedirs(OUT, exist_ok=True)
    import torch  # noqa: F401  (only for the include/library paths)
    from torch.utils import cpp_extension as ce

    inc = ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]
    common = [
        "nvcc", "-c", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "--expt-relaxed-constexpr", "-w",
        f"-DTORCH_EXTENSION_NAME={NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
        "-D_GLIBCXX_USE_CXX11_ABI=1",
    ] + [f"-I{p}" for p in inc]

    def one(src: str) -> str:
        obj = os.path.join(OUT, os.path.basename(src) + ".o")
        subprocess.run(common + [src, "-o", obj], check=True)
        return obj

    with ThreadPoolExecutor(max_workers=4) as ex:
        objs = list(ex.map(one, srcs))
    libs = ce.library_paths("cuda")
    link = ["g++", "-shared", "-o", target] + objs
    for p in libs:
        link += [f"-L{p}", f"-Wl,-rpath,{p}"]
    link += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    subprocess.run(link, check=True)
    if verbose:
        print(f"[build_ref] built {target}")
    return target


def load():
    """Import the built module (needs ``import torch`` first). Returns None if it was never built."""
    path = so_path()
    if not os.path.exists(path):
        return None
    import importlib.util

    import torch  # noqa: F401

    spec = importlib.util.spec_from_file_location(NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REFERENCE
    build(root, force="--force" in sys.argv)
