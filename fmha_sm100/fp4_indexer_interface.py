"""``fmha_sm100.fp4_indexer_interface``: the FP4 indexer names of the reference module
python/fmha_sm100/cute/fp4_indexer_interface.py, served by ``msa_b200.fp4_indexer``."""
from msa_b200.fp4_indexer import (fp4_indexer_block_scores, fp4_indexer_mma_scale_shape,  # noqa: F401
                                  fp4_indexer_mma_scale_storage_shape, fp4_indexer_mma_scale_storage_stride,
                                  fp4_indexer_mma_scale_stride, fp4_indexer_reorder_scales_for_mma_cute)

__all__ = ["fp4_indexer_block_scores", "fp4_indexer_reorder_scales_for_mma_cute", "fp4_indexer_mma_scale_shape",
           "fp4_indexer_mma_scale_stride", "fp4_indexer_mma_scale_storage_shape",
           "fp4_indexer_mma_scale_storage_stride"]
