"""Backend selection, kept for API compatibility with the reference (nsa/backend.py:8-60).

This package has ONE backend - the sm_100a CUDA library - so the functions below accept
the reference's names but only ever resolve to "cuda"; asking for "triton" raises."""
import os

BACKENDS = ("cuda",)
_ENV = "OMNIMEM_NSA_BACKEND"


def resolve_backend(name=None) -> str:
    name = (name or os.environ.get(_ENV) or "cuda").lower()
    if name != "cuda":
        raise ValueError(f"omnimem_b200 has a single backend ('cuda', sm_100a kernels); got {name!r}")
    return name


def get_backend() -> str:
    return "cuda"


def set_backend(name: str) -> str:
    return resolve_backend(name)
