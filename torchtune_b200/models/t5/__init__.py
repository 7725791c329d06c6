"""T5 encoder (text conditioning for diffusion models; parity: torchtune/models/t5/__init__.py)."""
from ._builders import T5Tokenizer, t5_encoder, t5_encoder_hf_to_tune, t5_tokenizer, t5_v1_1_xxl_encoder
from ._encoder import T5Encoder, T5EncoderLayer, T5EncoderRelativePositionBias, T5EncoderSelfAttention

__all__ = ["T5Encoder", "T5EncoderLayer", "T5EncoderRelativePositionBias", "T5EncoderSelfAttention", "T5Tokenizer", "t5_encoder", "t5_encoder_hf_to_tune", "t5_tokenizer", "t5_v1_1_xxl_encoder"]
