"""The reference's own CUDA append kernel, compiled from its checkout for the GPU tests.

TEST INFRASTRUCTURE ONLY: imported by the tests and the benchmark's reference legs, never by the
product package.

``build(reference_root)`` compiles ``csrc/kernels/paged_kv_cache.cu`` *where it lies* in a reference
checkout, together with ``ref_cuda_binding.cpp`` (a binding for that one launcher), into
``oracle/_ref/barqtrain_ref_paged.so`` for compute capability 10.0.  No reference source is copied; the
output directory is not under version control.  nvcc cross-compiles, so this runs on a machine
without a GPU; the shared object is then used wherever the checkout is absent.

``load()`` imports the built module (``None`` when it has not been built).  It exposes
``paged_kv_append_(key_cache, value_cache, seq_lens, key_states, value_states)`` exactly as the
reference's ``barqtrain_cuda`` module does (``csrc/src/bindings.cpp:74-75``).
"""

from __future__ import annotations

import importlib.util
import os
import subprocess
import sys
import sysconfig
from pathlib import Path
from typing import Optional

_HERE = Path(__file__).resolve().parent
_OUT_DIR = _HERE / "_ref"
_NAME = "barqtrain_ref_paged"
_OUT = _OUT_DIR / f"{_NAME}.so"
_KERNEL = Path("csrc") / "kernels" / "paged_kv_cache.cu"
_MODULE = None


def default_reference_root() -> Optional[Path]:
    """``$BARQTRAIN_REFERENCE``, else a directory ``reference`` beside this repository, else ``None``."""
    root = os.environ.get("BARQTRAIN_REFERENCE")
    if root:
        return Path(root)
    beside = _HERE.parent.parent / "reference"
    return beside if (beside / _KERNEL).exists() else None


def build(reference_root=None, force: bool = False) -> Optional[Path]:
    """Compile the reference kernel; returns the module path, or ``None`` when there is no checkout."""
    root = Path(reference_root) if reference_root else default_reference_root()
    if root is None or not (root / _KERNEL).exists():
        return _OUT if _OUT.exists() else None
    kernel = root / _KERNEL
    binding = _HERE / "ref_cuda_binding.cpp"
    newest = max(kernel.stat().st_mtime, binding.stat().st_mtime)
    if not force and _OUT.exists() and _OUT.stat().st_mtime >= newest:
        return _OUT
    import torch
    from torch.utils import cpp_extension

    _OUT_DIR.mkdir(parents=True, exist_ok=True)
    cuda_home = cpp_extension.CUDA_HOME or "/usr/local/cuda"
    includes = [f"-I{p}" for p in cpp_extension.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    abi = f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"
    common = includes + [abi, f"-DTORCH_EXTENSION_NAME={_NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H", "-O3", "-std=c++17"]
    obj_kernel, obj_binding = _OUT_DIR / "paged_kv_cache.o", _OUT_DIR / "ref_cuda_binding.o"
    nvcc = str(Path(cuda_home) / "bin" / "nvcc")
    subprocess.run([nvcc, "-c", str(kernel), "-o", str(obj_kernel), "-gencode", "arch=compute_100,code=sm_100",
                    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"] + common, check=True, capture_output=True, text=True)
    subprocess.run(["g++", "-c", str(binding), "-o", str(obj_binding), "-fPIC"] + common,
                   check=True, capture_output=True, text=True)
    lib_dirs = cpp_extension.library_paths("cuda")
    link = ["g++", "-shared", "-o", str(_OUT) + ".tmp", str(obj_kernel), str(obj_binding)]
    for d in lib_dirs:
        link += [f"-L{d}", f"-Wl,-rpath,{d}"]
    link += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    subprocess.run(link, check=True, capture_output=True, text=True)
    os.replace(str(_OUT) + ".tmp", _OUT)
    for obj in (obj_kernel, obj_binding):
        obj.unlink()
    return _OUT


def load():
    """The built module, or ``None`` when ``oracle/_ref`` holds no build."""
    global _MODULE
    if _MODULE is not None:
        return _MODULE
    if not _OUT.exists():
        return None
    import torch  # noqa: F401  (the module links against libtorch)

    spec = importlib.util.spec_from_file_location(_NAME, _OUT)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    sys.modules[_NAME] = module
    _MODULE = module
    return module
