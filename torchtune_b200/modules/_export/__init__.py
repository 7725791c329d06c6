"""Export-friendly module variants (parity: torchtune/modules/_export): same parameters and state-dict keys as the training
modules, but written only with plain, shape-static PyTorch ops (no custom kernels, no data-dependent Python control flow) so that
``torch.export`` can trace them for on-device runtimes."""
from ._position_embeddings import TiledTokenPositionalEmbedding, TilePositionalEmbedding, replace_tile_positional_embedding, replace_tiled_token_positional_embedding
from .attention import SDPA, MultiHeadAttention, replace_mha_with_inference_mha
from .kv_cache import KVCache

__all__ = ["KVCache", "MultiHeadAttention", "SDPA", "TilePositionalEmbedding", "TiledTokenPositionalEmbedding", "replace_mha_with_inference_mha",
           "replace_tile_positional_embedding", "replace_tiled_token_positional_embedding"]
