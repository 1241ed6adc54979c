"""B200-native sparse-attention forward path for sparse-wsi-vit.

Importing this package loads ``csrc/libswv_b200.so``; it raises ImportError if
the library has not been built (``python sparse_wsi_vit_b200/csrc/build.py``).
"""
from . import _lib  # noqa: F401  (fails loudly when the CUDA library is missing)
from .ops import (DSAAttentionFunction, LightningIndexerFunction, check_status, dsa_attention_gather,
                  dsa_attention_masked, dsa_indexer_topk, dsa_sparse_attention)
from .ops import block_sparse_attention, rope2d
from .modules import DeepSeekSparseAttention, DSAViTBlock, DSAViTSlideEncoder, IndexerProjection
from .static_modules import (BlockSparse2DViTBlock, BlockSparse2DViTSlideEncoder, BlockSparseAttention2D,
                             StaticSparseAttention, StaticSparseViTBlock, StaticSparseViTSlideEncoder)
from . import ingest, patterns, training

__all__ = [
    "DSAAttentionFunction", "LightningIndexerFunction", "check_status", "dsa_attention_gather",
    "dsa_attention_masked", "dsa_indexer_topk", "dsa_sparse_attention", "DeepSeekSparseAttention",
    "DSAViTBlock", "DSAViTSlideEncoder", "IndexerProjection", "block_sparse_attention", "rope2d", "patterns", "ingest", "training",
    "BlockSparseAttention2D", "BlockSparse2DViTBlock", "BlockSparse2DViTSlideEncoder", "StaticSparseAttention", "StaticSparseViTBlock", "StaticSparseViTSlideEncoder",
]
