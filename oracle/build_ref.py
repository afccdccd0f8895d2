"""Build recipe of the second judge: the reference's own code, compiled where it lies.

Test infrastructure, not product code: nothing under omnimem_b200/ imports or loads what this
writes.  Only tests/, __graft_entry__ and bench.py's baseline legs use it.

    python -m oracle.build_ref [--force]

writes, into the git-ignored folder oracle/_ref/ (which still travels to the GPU machine):

* ``omnimem_nsa_ref.so`` - the reference's NSA CUDA extension (bindings.cpp, topk.cu,
  ptr_table.cu, selection_fwd.cu, selection_bwd.cu, inverted_index.cu of
  src/omnimem/nsa/cuda_backend/csrc, flags of cuda_backend/_loader.py:15-34) compiled for
  sm_100a straight from the read-only reference tree with torch's cpp_extension - no source is
  copied.  It registers ``torch.ops.omnimem_nsa.*`` when loaded with torch.ops.load_library, so
  it must be loaded in a process of its own (tests/ref_cuda_runner.py): the product registers
  the same operator names from Python.
* ``omnimem_block_kv_ref*.so`` - the reference's block-KV pybind module (K1 gather, K2 range,
  K3 dedup; cuda_backend/_block_kv_loader.py:13-23).

The reference tree exists only in the build container.  Without it the recipe does nothing
and reports what is already built; on the GPU machine the prebuilt files are used as they are.
"""
from __future__ import annotations

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
REFERENCE = os.environ.get("OMNIMEM_REFERENCE", "/root/reference")
CSRC = os.path.join(REFERENCE, "src", "omnimem", "nsa", "cuda_backend", "csrc")
NSA_LIB = os.path.join(OUT, "omnimem_nsa_ref.so")
BLOCK_KV_NAME = "omnimem_block_kv_ref"

NSA_SOURCES = ("bindings.cpp", "topk.cu", "ptr_table.cu", "selection_fwd.cu", "selection_bwd.cu", "inverted_index.cu")
NSA_CUDA_FLAGS = ["-O3", "-std=c++17", "--expt-relaxed-constexpr", "--expt-extended-lambda", "-lineinfo",
                  "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
                  "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__"]
BLOCK_KV_SOURCES = ("block_kv_bindings.cpp", "block_kv_gather.cu", "block_kv_range.cu", "block_kv_dedup.cu")
BLOCK_KV_CUDA_FLAGS = ["-O3", "-std=c++17", "-lineinfo"]


def block_kv_library():
    """Path of the built block-KV module, or None."""
    if not os.path.isdir(OUT):
        return None
    for f in sorted(os.listdir(OUT)):
        if f.startswith(BLOCK_KV_NAME) and f.endswith(".so"):
            return os.path.join(OUT, f)
    return None


def available() -> dict:
    return {"nsa": NSA_LIB if os.path.exists(NSA_LIB) else None, "block_kv": block_kv_library()}


def _load(name, sources, cuda_flags, python_module, build_dir):
    from torch.utils import cpp_extension
    os.makedirs(build_dir, exist_ok=True)
    old = os.environ.get("TORCH_CUDA_ARCH_LIST")
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
    try:
        cpp_extension.load(name=name, sources=[os.path.join(CSRC, s) for s in sources],
                           extra_cflags=["-O3", "-std=c++17"], extra_cuda_cflags=list(cuda_flags),
                           extra_include_paths=[CSRC], build_directory=build_dir, verbose=False, with_cuda=True,
                           is_python_module=python_module, keep_intermediates=False)
    finally:
        if old is None:
            os.environ.pop("TORCH_CUDA_ARCH_LIST", None)
        else:
            os.environ["TORCH_CUDA_ARCH_LIST"] = old


def build(force: bool = False) -> dict:
    """Compile what is missing (everything with `force`); returns available()."""
    if not os.path.isdir(CSRC):
        return available()
    import shutil
    os.makedirs(OUT, exist_ok=True)
    if force or not os.path.exists(NSA_LIB):
        bd = os.path.join(OUT, "build_nsa")
        _load("omnimem_nsa_ref", NSA_SOURCES, NSA_CUDA_FLAGS, False, bd)
        shutil.copyfile(os.path.join(bd, "omnimem_nsa_ref.so"), NSA_LIB)
        shutil.rmtree(bd, ignore_errors=True)
    if force or block_kv_library() is None:
        bd = os.path.join(OUT, "build_block_kv")
        _load(BLOCK_KV_NAME, BLOCK_KV_SOURCES, BLOCK_KV_CUDA_FLAGS, True, bd)
        shutil.copyfile(os.path.join(bd, BLOCK_KV_NAME + ".so"), os.path.join(OUT, BLOCK_KV_NAME + ".so"))
        shutil.rmtree(bd, ignore_errors=True)
    return available()


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
