"""The reference's own CPU path for the paged KV cache, byte-compiled from its checkout.

TEST INFRASTRUCTURE ONLY: imported by the tests and the benchmark's reference legs, never by the
product package.

The reference's CPU implementation of the path is pure Python: ``BarqPagedKVCacheLayer`` with
``_python_append`` and ``current_tensors`` in ``python/barqtrain/kv_cache.py`` (37-194), plus the loader
it imports (``python/barqtrain/_ffi.py``).  ``build(reference_root)`` byte-compiles those two files
*where they lie* in a reference checkout into ``oracle/_ref/barqtrain_ref_py_<tag>/*.code`` (marshalled
code objects; not named ``.pyc``, which tools that copy a working tree tend to leave behind) - the
Python counterpart of compiling a C reference into a shared object.  No reference source is copied and
the output directory is not under version control; it travels with the working tree to machines that
have no checkout, which must run the same Python minor version that compiled it (the folder name carries
it).

``load()`` executes those code objects as the modules ``barqtrain._ffi`` and ``barqtrain.kv_cache`` with the
reference's native backend disabled (``BARQTRAIN_AUTO_BUILD=0``, so ``append`` takes ``_python_append``,
kv_cache.py:75-91), or returns ``None`` when they are not there.  ``barqtrain`` itself is a bare namespace
module: the reference's ``barqtrain/__init__.py``, which pulls in its training stack, is not part of the
path and is not compiled.
"""

from __future__ import annotations

import marshal
import os
import sys
import types
from pathlib import Path
from typing import Optional

_HERE = Path(__file__).resolve().parent
_TAG = f"py{sys.version_info.major}{sys.version_info.minor}"
_OUT_DIR = _HERE / "_ref" / f"barqtrain_ref_py_{_TAG}"
_FILES = ("_ffi.py", "kv_cache.py")            # in import order
_MODULE = None


def default_reference_root() -> Optional[Path]:
    """``$BARQTRAIN_REFERENCE``, else a directory ``reference`` beside this repository, else ``None``."""
    root = os.environ.get("BARQTRAIN_REFERENCE")
    if root:
        return Path(root)
    beside = _HERE.parent.parent / "reference"
    return beside if (beside / "python" / "barqtrain" / "kv_cache.py").exists() else None


def _out(name: str) -> Path:
    return _OUT_DIR / (Path(name).stem + ".code")


def built() -> bool:
    return all(_out(f).exists() for f in _FILES)


def build(reference_root=None, force: bool = False) -> Optional[Path]:
    """Byte-compile the reference's two files; returns the output folder, or ``None`` when there is neither a
    checkout nor an earlier build."""
    root = Path(reference_root) if reference_root else default_reference_root()
    if root is None or not (root / "python" / "barqtrain" / "kv_cache.py").exists():
        return _OUT_DIR if built() else None
    _OUT_DIR.mkdir(parents=True, exist_ok=True)
    for name in _FILES:
        src = root / "python" / "barqtrain" / name
        out = _out(name)
        if force or not out.exists() or out.stat().st_mtime < src.stat().st_mtime:
            code = compile(src.read_bytes(), f"<reference>/python/barqtrain/{name}", "exec", dont_inherit=True)
            out.write_bytes(marshal.dumps(code))
    return _OUT_DIR


def load():
    """The reference's ``barqtrain.kv_cache`` module (CPU path only), or ``None`` when nothing was built."""
    global _MODULE
    if _MODULE is not None:
        return _MODULE
    if not built():
        return None
    if "barqtrain" in sys.modules and not getattr(sys.modules["barqtrain"], "_barq_reference_bytecode", False):
        raise RuntimeError("another `barqtrain` package is already imported in this process")
    os.environ["BARQTRAIN_AUTO_BUILD"] = "0"         # no native build: append takes the reference's CPU loop
    package = types.ModuleType("barqtrain")
    package.__path__ = []                            # a package with nothing to find on disk
    package._barq_reference_bytecode = True
    sys.modules["barqtrain"] = package
    module = None
    for name in _FILES:
        stem = Path(name).stem
        module = types.ModuleType(f"barqtrain.{stem}")
        module.__file__ = str(_out(name))
        module.__package__ = "barqtrain"
        sys.modules[module.__name__] = module
        setattr(package, stem, module)
        exec(marshal.loads(_out(name).read_bytes()), module.__dict__)
    _MODULE = module
    return _MODULE
