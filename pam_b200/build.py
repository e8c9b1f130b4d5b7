"""Builds ``pam_b200/libpam_b200.so`` — every CUDA source under ``pam_b200/csrc`` compiled for
sm_100a with nvcc and linked into one C-ABI shared library (declared in ``include/pam_b200.h``).

    python -m pam_b200.build [--force] [--verbose]

The library does not depend on torch.  ``-fmad=false`` keeps nvcc from fusing a multiply into a
following add: the PAM kernels reproduce the reference's roundings operation by operation and
use explicit fused multiply-adds only where the reference's build does.
"""
import concurrent.futures
import pathlib
import shutil
import subprocess
import sys

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libpam_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false", "-Xcompiler", "-fPIC", "-Xcompiler", "-O2",
]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not pathlib.Path(exe).exists():
        raise RuntimeError("nvcc not found: pam_b200 needs the CUDA toolkit to build its kernels")
    return exe


def _stale(target, deps):
    return not target.exists() or any(d.stat().st_mtime > target.stat().st_mtime for d in deps)


def build(force=False, verbose=False):
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "pam_b200.h", pathlib.Path(__file__)]
    OBJ.mkdir(exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=8) as pool:
            for cmd, res in zip(jobs, pool.map(lambda c: subprocess.run(c, capture_output=True, text=True), jobs)):
                if verbose or res.returncode:
                    sys.stderr.write(res.stdout + res.stderr)
                if res.returncode:
                    raise RuntimeError("nvcc failed: " + " ".join(cmd))
    objs = [OBJ / (s.stem + ".o") for s in sources]
    if force or jobs or _stale(LIB, objs):
        subprocess.check_call([nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-gencode",
                               "arch=compute_100a,code=sm_100a"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
