"""TEST INFRASTRUCTURE — builds the CPU oracle libraries.

    python oracle/build.py            # liboracle (+ the reference build when the sources exist)

* ``oracle/libpam_oracle.so``  — the C restatement (pam_oracle.c), gcc -O2 -fopenmp.
* ``oracle/_ref/libpam_ref.so`` — the reference's OWN scalar functions, lines 15-136 of
  pam/cuda_kernels.cu, compiled for the host from where they lie.  The lines are streamed
  through a pipe between ref_prelude.h and array_loops.inc straight into g++; no reference
  source is written into this repository.  Skipped when the reference tree is not mounted
  (e.g. on a GPU box, which uses the prebuilt file).

Neither library is part of the shipped package: only tests, the smoke check and the benchmark's
CPU-baseline leg load them.
"""
import os
import pathlib
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
REF_CU = pathlib.Path(os.environ.get("PAM_REFERENCE_ROOT", "/root/reference")) / "pam" / "cuda_kernels.cu"
# The scalar functions of the reference file (first to last line, inclusive).
REF_FIRST, REF_LAST = 15, 136

CFLAGS = ["-O2", "-fPIC", "-shared", "-fopenmp", "-fno-fast-math", "-ffp-contract=off"]


def _newer(target: pathlib.Path, *sources: pathlib.Path) -> bool:
    return target.exists() and all(target.stat().st_mtime >= s.stat().st_mtime for s in sources)


def build_oracle(force: bool = False) -> pathlib.Path:
    out = HERE / "libpam_oracle.so"
    srcs = [HERE / "pam_oracle.c", HERE / "pam_scalar_oracle.h", HERE / "array_loops.inc"]
    if force or not _newer(out, *srcs):
        subprocess.check_call(["gcc", "-std=c11", *CFLAGS, "-o", str(out), str(srcs[0]), "-lm"], cwd=HERE)
    return out


def build_ref(force: bool = False):
    """Returns the path of the reference build, or None when the reference is not available."""
    out = HERE / "_ref" / "libpam_ref.so"
    if not REF_CU.exists():
        return out if out.exists() else None
    srcs = [HERE / "ref_prelude.h", HERE / "array_loops.inc", REF_CU]
    if force or not _newer(out, *srcs):
        out.parent.mkdir(exist_ok=True)
        lines = REF_CU.read_text().splitlines(keepends=True)[REF_FIRST - 1:REF_LAST]
        unit = (HERE / "ref_prelude.h").read_text() + "".join(lines) + (HERE / "array_loops.inc").read_text()
        subprocess.run(["g++", "-std=c++17", "-x", "c++", *CFLAGS, "-o", str(out), "-"],
                       input=unit.encode(), check=True, cwd=HERE)
    return out


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_oracle(force))
    print(build_ref(force))
