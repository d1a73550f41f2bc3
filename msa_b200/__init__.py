"""msa_b200: B200-native (sm_100a) kernels for the MSA block-sparse attention
hot path behind the reference's Python API names."""
from .api import (PlanInfo, fmha_sm100, fmha_sm100_plan, plan_status, sparse_topk_select)  # noqa: F401
from .api import fp8_pv_precision, get_fp8_pv_precision, set_fp8_pv_precision  # noqa: F401
from .quant import (Nvfp4QuantizedTensor, dequantize_nvfp4_128x4, quantize_bf16_to_nvfp4_128x4,  # noqa: F401
                    quantize_fp8_per_tensor, quantize_kv_bf16_to_nvfp4_128x4)
from .sparse import (SparseDecodePagedAttentionWrapper, build_k2q_csr, k2q_csr_to_lists, k2q_csr_to_q2k,  # noqa: F401
                     sparse_atten_func, sparse_atten_nvfp4_kv_func, sparse_decode_atten_func, sparse_prefill_nvfp4)
from .host_pipeline import HostPrefillPipeline  # noqa: F401
from .fp4_indexer import (fp4_indexer_block_scores, fp4_indexer_mma_scale_shape,  # noqa: F401
                          fp4_indexer_mma_scale_storage_shape, fp4_indexer_mma_scale_storage_stride,
                          fp4_indexer_mma_scale_stride, fp4_indexer_reorder_scales_for_mma,
                          fp4_indexer_reorder_scales_for_mma_cute)
from .kv_cache import absmax_bf16, append_kv_fp8, append_kv_nvfp4  # noqa: F401
from .shard import (gather_heads, head_shard, request_cost, scatter_rows, shard_batch, shard_kv_heads,  # noqa: F401
                    shard_requests)
from ._lib import MsaError, build_library, get_lib  # noqa: F401

__version__ = "0.1.0"
