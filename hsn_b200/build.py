"""Builds ``hsn_b200/lib/libhsn_window_b200.so`` from ``hsn_b200/csrc`` with nvcc for sm_100a.

The library is a plain C-ABI shared object (``include/hsn_window_b200.h``); nothing here needs a
GPU: nvcc cross-compiles. Run ``python -m hsn_b200.build`` (or ``__graft_entry__.build()``).
It plays the role of the reference's ``scripts/build_window_kernels.py`` and
``scripts/build_cuda_extension.py`` (a fatbin plus a host extension there; one library here) and,
like them, writes a manifest with the sources' SHA-256 next to the artifact.
"""

from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
ROOT = PACKAGE.parent
CSRC = PACKAGE / "csrc"
LIB_DIR = PACKAGE / "lib"
LIBRARY = LIB_DIR / "libhsn_window_b200.so"
MANIFEST = LIB_DIR / "window_build.json"
SOURCES = ("api.cu", "ops_kernels.cu", "sweep_kernels.cu", "window_fwd.cu", "window_bwd.cu", "window_rows.cu", "window_rows_bwd.cu", "selftest.cu", "prologue.cu", "trainer.cu", "decode.cu", "units.cu", "scorer.cu", "tail.cu", "gate.cu", "messages.cu")
HEADERS = ("common.cuh", "select.cuh", "stage.cuh", "umma.cuh", "host_util.h", "rows.cuh", "mma_tiles.cuh")
ARCH = ("-gencode", "arch=compute_100a,code=sm_100a")


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found: the window kernels need the CUDA toolkit to build")
    return found


def _sha(path: Path) -> str:
    return hashlib.sha256(path.read_bytes()).hexdigest()


def source_hashes() -> dict[str, str]:
    files = [CSRC / n for n in (*SOURCES, *HEADERS)] + [ROOT / "include" / "hsn_window_b200.h", ROOT / "include" / "hsn_trainer_b200.h", ROOT / "include" / "hsn_units_b200.h", ROOT / "include" / "hsn_scorer_b200.h", ROOT / "include" / "hsn_tail_b200.h", ROOT / "include" / "hsn_gate_b200.h", ROOT / "include" / "hsn_messages_b200.h"]
    return {str(f.relative_to(ROOT)): _sha(f) for f in files}


def up_to_date() -> bool:
    if not LIBRARY.is_file() or not MANIFEST.is_file():
        return False
    try:
        manifest = json.loads(MANIFEST.read_text())
    except json.JSONDecodeError:
        return False
    return manifest.get("sources") == source_hashes() and manifest.get("library_sha256") == _sha(LIBRARY)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``.cu`` of ``csrc`` for sm_100a and link the shared library."""
    if not force and up_to_date():
        return LIBRARY
    LIB_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()
    objects = []
    flags = ["-O3", "-std=c++17", "-lineinfo", *ARCH, "-Xcompiler", "-fPIC", "-Xptxas", "-v" if verbose else "-O3"]
    flags += os.environ.get("HSNW_NVCC_FLAGS", "").split()  # e.g. -DHSNW_TRACE for the phase timestamps
    jobs = []
    for name in SOURCES:
        obj = LIB_DIR / (Path(name).stem + ".o")
        cmd = [nvcc, *flags, "-c", str(CSRC / name), "-o", str(obj)]
        jobs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(str(obj))
    for name, proc in jobs:
        out, _ = proc.communicate()
        if verbose or proc.returncode:
            sys.stderr.write(out)
        if proc.returncode:
            raise RuntimeError(f"nvcc failed on {name}")
    link = [nvcc, *ARCH, "-shared", "-o", str(LIBRARY), *objects, "-lcudart"]
    subprocess.run(link, check=True)
    MANIFEST.write_text(
        json.dumps({"sources": source_hashes(), "library_sha256": _sha(LIBRARY), "arch": "sm_100a"}, indent=1)
    )
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv or os.environ.get("HSNW_VERBOSE") == "1"))
