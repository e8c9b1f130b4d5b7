"""TEST / BENCHMARK INFRASTRUCTURE — builds the reference's own CUDA kernels for sm_100a.

    python baseline/build_ref.py [--force]

The reference's ``pam/cuda_kernels.cu`` does not compile against current PyTorch as shipped: ten
``AT_DISPATCH_FLOATING_TYPES(X.type(), ...)`` sites pass the deprecated ``Tensor::type()``.  This
recipe reads the file where it lies in the mounted reference tree, rewrites those ten
``.type()`` tokens to ``.scalar_type()`` in memory, writes the result to a temporary directory
outside this repository, and compiles it as a PyTorch extension with the reference's own flags
(``-std=c++17 -O3``, pam/cuda_bindings.py:15-25) for sm_100a only.  The only thing kept is the
compiled module ``baseline/_ref/pam_ref_cuda_kernels.so`` (git-ignored).  No reference source is
written into the repository.

The module serves two purposes, neither on the product path:
  * the kernel to beat: ``bench.py`` times its ``pam_matmul_fwd`` on the same inputs in the same run;
  * an on-GPU bit-exact oracle for whole outputs (``tests/test_gpu_ref_kernel.py``).

Skipped (returns the existing file or None) when the reference tree is not mounted.
"""
import importlib.util
import os
import pathlib
import re
import shutil
import sys
import tempfile

HERE = pathlib.Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
NAME = "pam_ref_cuda_kernels"
OUT = OUT_DIR / f"{NAME}.so"
REF_CU = pathlib.Path(os.environ.get("PAM_REFERENCE_ROOT", "/root/reference")) / "pam" / "cuda_kernels.cu"


def build(force: bool = False, verbose: bool = False):
    if not REF_CU.exists():
        return OUT if OUT.exists() else None
    if OUT.exists() and not force and OUT.stat().st_mtime >= REF_CU.stat().st_mtime:
        return OUT
    text = REF_CU.read_text()
    patched, count = re.subn(r"(AT_DISPATCH_FLOATING_TYPES\(\s*\w+)\.type\(\)", r"\1.scalar_type()", text)
    if count != 10:
        raise RuntimeError(f"expected 10 dispatch sites to patch in {REF_CU}, found {count}")
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
    from torch.utils import cpp_extension
    OUT_DIR.mkdir(exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="pam_ref_build_") as tmp:
        src = pathlib.Path(tmp) / "cuda_kernels_patched.cu"
        src.write_text(patched)
        build_dir = pathlib.Path(tmp) / "build"
        build_dir.mkdir()
        cpp_extension.load(name=NAME, sources=[str(src)], extra_cflags=["-std=c++17", "-O3"],
                           extra_cuda_cflags=["-std=c++17", "-O3"], build_directory=str(build_dir),
                           verbose=verbose, is_python_module=False)
        shutil.copy2(build_dir / f"{NAME}.so", OUT)
    return OUT


def load():
    """Imports the built module (torch must be importable; the module needs a CUDA device to run).
    Returns None when it was never built."""
    if not OUT.exists():
        return None
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location(NAME, OUT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
