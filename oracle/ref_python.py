"""The reference's own CPU path for the paged KV cache, byte-compiled from its checkout.

TEST INFRASTRUCTURE ONLY: imported by the tests and the benchmark's reference legs, never by the
product package.

The reference's CPU implementation of the path is pure Python: ``BarqPagedKVCacheLayer`` with
``_python_append`` and ``current_tensors`` in ``python/barqtrain/kv_cache.py`` (37-194), plus the loader
it imports (``python/barqtrain/_ffi.py``).  ``build(reference_root)`` byte-compiles those two files
*where they lie* in a reference checkout into ``oracle/_ref/barqtrain_ref_py/barqtrain/*.pyc`` - the
Python counterpart of compiling a C reference into a shared object.  No reference source is copied and
the output directory is not under version control; it travels with the working tree to machines that
have no checkout, which must run the same Python minor version that compiled it (the file name carries
it).

``load()`` imports ``barqtrain.kv_cache`` from those files with the reference's native backend
disabled (``BARQTRAIN_AUTO_BUILD=0``, so ``append`` takes ``_python_append``, kv_cache.py:75-91), or
returns ``None`` when they are not there.  The package is loaded as a bare namespace: the reference's
``barqtrain/__init__.py``, which pulls in its training stack, is not part of the path and is not
compiled.
"""

from __future__ import annotations

import importlib
import os
import py_compile
import sys
from pathlib import Path
from typing import Optional

_HERE = Path(__file__).resolve().parent
_TAG = f"py{sys.version_info.major}{sys.version_info.minor}"
_OUT_DIR = _HERE / "_ref" / f"barqtrain_ref_py_{_TAG}"
_FILES = ("kv_cache.py", "_ffi.py")
_MODULE = None


def default_reference_root() -> Optional[Path]:
    """``$BARQTRAIN_REFERENCE``, else a directory ``reference`` beside this repository, else ``None``."""
    root = os.environ.get("BARQTRAIN_REFERENCE")
    if root:
        return Path(root)
    beside = _HERE.parent.parent / "reference"
    return beside if (beside / "python" / "barqtrain" / "kv_cache.py").exists() else None


def built() -> bool:
    return all((_OUT_DIR / "barqtrain" / (Path(f).stem + ".pyc")).exists() for f in _FILES)


def build(reference_root=None, force: bool = False) -> Optional[Path]:
    """Byte-compile the reference's two files; returns the output folder, or ``None`` when there is neither a
    checkout nor an earlier build."""
    root = Path(reference_root) if reference_root else default_reference_root()
    if root is None or not (root / "python" / "barqtrain" / "kv_cache.py").exists():
        return _OUT_DIR if built() else None
    pkg = _OUT_DIR / "barqtrain"
    pkg.mkdir(parents=True, exist_ok=True)
    for name in _FILES:
        src = root / "python" / "barqtrain" / name
        out = pkg / (Path(name).stem + ".pyc")
        if force or not out.exists() or out.stat().st_mtime < src.stat().st_mtime:
            # unchecked-hash pyc: valid wherever the file goes, whatever the source's timestamp was
            py_compile.compile(str(src), cfile=str(out), dfile=f"<reference>/python/barqtrain/{name}", doraise=True,
                               invalidation_mode=py_compile.PycInvalidationMode.UNCHECKED_HASH)
    return _OUT_DIR


def load():
    """The reference's ``barqtrain.kv_cache`` module (CPU path only), or ``None`` when nothing was built."""
    global _MODULE
    if _MODULE is not None:
        return _MODULE
    if not built():
        return None
    if "barqtrain" in sys.modules and not str(getattr(sys.modules["barqtrain"], "__path__", "")).count(str(_OUT_DIR)):
        raise RuntimeError("another `barqtrain` package is already imported in this process")
    os.environ["BARQTRAIN_AUTO_BUILD"] = "0"         # no native build: append takes the reference's CPU loop
    sys.path.insert(0, str(_OUT_DIR))
    try:
        _MODULE = importlib.import_module("barqtrain.kv_cache")
    finally:
        sys.path.remove(str(_OUT_DIR))
    return _MODULE
