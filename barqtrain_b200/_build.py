"""Build recipe for ``libbarqkv.so`` (sm_100a only, plain nvcc, built in-tree)."""

from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path
from typing import List, Optional

PACKAGE_DIR = Path(__file__).resolve().parent
SOURCE = PACKAGE_DIR / "csrc" / "barqkv.cu"
HEADER_DIR = PACKAGE_DIR.parent / "include"
LIBRARY = PACKAGE_DIR / "lib" / "libbarqkv.so"
TUNING_LIBRARY = PACKAGE_DIR / "lib" / "libbarqkv_tuning.so"     # -DBARQKV_TUNING: adds barqkv_set_tuning, for sweeps


def detect_cuda_home() -> Optional[str]:
    """CUDA_HOME / CUDA_PATH first, then nvcc on PATH, then the usual install prefixes."""
    for env_name in ("CUDA_HOME", "CUDA_PATH"):
        home = os.environ.get(env_name)
        if home and Path(home).exists():
            return home
    nvcc = shutil.which("nvcc")
    if nvcc:
        return str(Path(nvcc).resolve().parents[1])
    for candidate in ("/usr/local/cuda", "/opt/cuda"):
        if Path(candidate).exists():
            return candidate
    return None


def nvcc_command(output: Path = LIBRARY, verbose_ptxas: bool = False, tuning: bool = False) -> List[str]:
    home = detect_cuda_home()
    if home is None:
        raise RuntimeError("no CUDA toolkit found (set CUDA_HOME)")
    cmd = [
        str(Path(home) / "bin" / "nvcc"),
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-lineinfo", "-O3", "-std=c++17",
        "-shared", "-Xcompiler", "-fPIC",
        f"-I{HEADER_DIR}",
        "-o", str(output), str(SOURCE),
    ]
    if verbose_ptxas:
        cmd[1:1] = ["-Xptxas", "-v"]
    if tuning:
        cmd[1:1] = ["-DBARQKV_TUNING"]
    return cmd


def is_stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    deps = [SOURCE, SOURCE.parent / "paged_attention.cuh", SOURCE.parent / "host_table.cuh", HEADER_DIR / "barqkv.h", HEADER_DIR / "barqkv_experimental.h"]
    return any(d.exists() and d.stat().st_mtime > built for d in deps)


def build_native(force: bool = False, verbose: bool = False, tuning: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources; returns its path.
    ``tuning=True`` builds the experiment variant (always) beside it."""
    if tuning:
        TUNING_LIBRARY.parent.mkdir(parents=True, exist_ok=True)
        scratch = TUNING_LIBRARY.with_name(f"{TUNING_LIBRARY.name}.{os.getpid()}.tmp")
        proc = subprocess.run(nvcc_command(output=scratch, tuning=True), capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
        os.replace(scratch, TUNING_LIBRARY)
        return TUNING_LIBRARY
    if not force and not is_stale():
        return LIBRARY
    if not SOURCE.exists():
        raise RuntimeError(f"CUDA source missing: {SOURCE}")
    LIBRARY.parent.mkdir(parents=True, exist_ok=True)
    # Build beside the target and rename: several processes (one per GPU) may get here at once, and a
    # reader must never open a half-written library.
    scratch = LIBRARY.with_name(f"{LIBRARY.name}.{os.getpid()}.tmp")
    try:
        proc = subprocess.run(nvcc_command(output=scratch, verbose_ptxas=verbose), capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
        os.replace(scratch, LIBRARY)
    finally:
        if scratch.exists():
            scratch.unlink()
    if verbose:
        print(proc.stdout + proc.stderr)
    return LIBRARY
