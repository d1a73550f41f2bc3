"""Import-compatible alias of the reference package name: ``import fmha_sm100`` (python/fmha_sm100/__init__.py of
MiniMax-AI/MSA) resolves to the sm_100a kernels of ``msa_b200``.  Same public names:
``fmha_sm100_plan`` / ``fmha_sm100`` / ``sparse_topk_select`` at the top level, the CSR-driven and decode entry
points lazily from ``fmha_sm100.sparse`` (the reference keeps them off the import path of its root package the
same way).
"""
from msa_b200 import fmha_sm100, fmha_sm100_plan, sparse_topk_select  # noqa: F401

_SPARSE_EXPORTS = frozenset({
    "sparse_atten_func", "sparse_atten_nvfp4_kv_func", "sparse_decode_atten_func",
    "SparseDecodePagedAttentionWrapper", "build_k2q_csr",
})

__all__ = ["fmha_sm100_plan", "fmha_sm100", "sparse_topk_select", *sorted(_SPARSE_EXPORTS)]


def __getattr__(name):
    if name in _SPARSE_EXPORTS:
        from . import sparse as _sparse
        return getattr(_sparse, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
