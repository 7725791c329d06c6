"""Registers the T5 encoder converter with the checkpoint codec registry."""
from ._builders import t5_encoder_hf_to_tune


def _register() -> None:
    from ...training.checkpointing._codecs import register_hf_codec
    from ...training.checkpointing._utils import ModelType

    def _no_export(sd, cfg):
        raise NotImplementedError("T5 encoder checkpoints are read-only (the decoder half is not modelled)")

    register_hf_codec(ModelType.T5_ENCODER, lambda sd, cfg: t5_encoder_hf_to_tune(sd), _no_export)


_register()
