"""``fmha_sm100.sparse`` of the reference (python/fmha_sm100/sparse.py): the CSR-driven sparse prefill, the paged
FP8 decode entry points and the NVFP4 quantisation helpers, served by ``msa_b200``."""
from msa_b200.quant import (Nvfp4QuantizedTensor, dequantize_nvfp4_128x4 as dequantize_nvfp4_128x4_to_bf16,  # noqa: F401
                            quantize_bf16_to_nvfp4_128x4, quantize_kv_bf16_to_nvfp4_128x4)
from msa_b200.sparse import (SparseDecodePagedAttentionWrapper, build_k2q_csr, sparse_atten_func,  # noqa: F401
                             sparse_atten_nvfp4_kv_func, sparse_decode_atten_func)
