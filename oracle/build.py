"""TEST INFRASTRUCTURE — builds the CPU oracle libraries.

    python oracle/build.py            # liboracle (+ the reference build when the sources exist)

* ``oracle/libpam_oracle.so``  — the C restatement (pam_oracle.c), gcc -O2 -fopenmp.
* ``oracle/_ref/libpam_ref.so`` — the reference's OWN scalar functions, lines 15-136 of
  pam/cuda_kernels.cu, compiled for the host from where they lie.  The lines are streamed
  through a pipe between ref_prelude.h and array_loops.inc straight into g++; no reference
  source is written into this repository.  Skipped when the reference tree is not mounted
  (e.g. on a GPU box, which uses the prebuilt file).
* ``oracle/_ref/pam_native/`` — the reference's own CPU implementation (pam/native.py and the
  pam/utils.py it imports), staged unmodified from the mounted tree into this git-ignored build
  folder so that the benchmark's CPU arm can time the real thing on a machine where the tree is
  not mounted.  ``load_native()`` imports it; nothing under ``oracle/_ref`` is ever committed.

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


NATIVE_FILES = ("native.py", "utils.py")


def build_native(force: bool = False):
    """Stages the reference's native PyTorch path; returns its folder, or None when neither the
    reference tree nor an earlier staging exists."""
    out = HERE / "_ref" / "pam_native"
    src_dir = REF_CU.parent
    have = all((out / f).exists() for f in NATIVE_FILES)
    if not all((src_dir / f).exists() for f in NATIVE_FILES):
        return out if have else None
    if force or not have or any((src_dir / f).stat().st_mtime > (out / f).stat().st_mtime for f in NATIVE_FILES):
        out.mkdir(parents=True, exist_ok=True)
        for f in NATIVE_FILES:
            (out / f).write_bytes((src_dir / f).read_bytes())
        (out / "__init__.py").write_text("")
    return out


def load_native():
    """The staged reference module ``native`` (pam/native.py), or None when it was never staged."""
    import importlib.util
    out = HERE / "_ref" / "pam_native"
    if not all((out / f).exists() for f in NATIVE_FILES):
        return None
    name = "pam_reference_native"
    if name in sys.modules:
        return sys.modules[name].native
    spec = importlib.util.spec_from_file_location(name, out / "__init__.py", submodule_search_locations=[str(out)])
    pkg = importlib.util.module_from_spec(spec)
    sys.modules[name] = pkg
    spec.loader.exec_module(pkg)
    import importlib
    pkg.native = importlib.import_module(name + ".native")
    return pkg.native


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_oracle(force))
    print(build_ref(force))
    print(build_native(force))
