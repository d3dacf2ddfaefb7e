"""Build recipe of libSOFIE_cuda.so (nvcc, sm_100a only) -- in-tree, no JIT cache.

The library is the product's only compute back end; nothing here falls back to a CPU path.
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = Path(__file__).resolve().parent / "csrc"
LIBDIR = Path(__file__).resolve().parent / "lib"
LIB = LIBDIR / "libSOFIE_cuda.so"
STAMP = LIBDIR / "libSOFIE_cuda.stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-ffp-contract=off", "-I", str(ROOT / "include"), "-I", str(CSRC),
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: libSOFIE_cuda cannot be built")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _fingerprint() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [ROOT / "include" / "sofie_cuda.h"]):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu under csrc/ into one shared library. Re-uses an up-to-date build."""
    fp = _fingerprint()

    def current():
        return not force and LIB.exists() and STAMP.exists() and STAMP.read_text().strip() == fp
    if current():
        return LIB
    LIBDIR.mkdir(parents=True, exist_ok=True)
    # one builder at a time: the ranks of a multi-GPU job all arrive here; the first compiles, the rest wait
    with open(LIBDIR / ".build.lock", "a+") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if current():
                return LIB
            return _compile_and_link(fp, verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _compile_and_link(fp: str, verbose: bool) -> Path:
    objdir = LIBDIR / "obj"
    objdir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    procs = []
    objs = []
    for src in sources():
        obj = objdir / (src.stem + ".o")
        objs.append(str(obj))
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if verbose and out:
            print(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{out}")
    tmp = LIB.with_name(f".{LIB.name}.{os.getpid()}.tmp")
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", *objs, "-o", str(tmp), "-lcudart"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise RuntimeError(f"link of {LIB.name} failed:\n{r.stdout}")
    os.replace(tmp, LIB)
    STAMP.write_text(fp)
    return LIB


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
