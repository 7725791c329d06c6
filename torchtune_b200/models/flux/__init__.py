"""Flux.1 autoencoder (parity: torchtune/models/flux/__init__.py)."""
from typing import List

from ._autoencoder import FluxAutoencoder, FluxDecoder, FluxEncoder
from ._convert_weights import flux_ae_hf_to_tune


def flux_1_autoencoder(resolution: int = 256, ch_in: int = 3, ch_out: int = 3, ch_base: int = 128, ch_mults: List[int] = (1, 2, 4, 4), ch_z: int = 16, n_layers_per_resample_block: int = 2,
                       scale_factor: float = 0.3611, shift_factor: float = 0.1159) -> FluxAutoencoder:
    """The autoencoder released with Flux.1: 8× spatial down-sampling to 16 latent channels; the decoder has one
    more ResNet layer per resolution than the encoder."""
    channels = [ch_base * m for m in ch_mults]
    encoder = FluxEncoder(ch_in=ch_in, ch_z=ch_z, channels=channels, n_layers_per_down_block=n_layers_per_resample_block, scale_factor=scale_factor, shift_factor=shift_factor)
    decoder = FluxDecoder(ch_out=ch_out, ch_z=ch_z, channels=list(reversed(channels)), n_layers_per_up_block=n_layers_per_resample_block + 1, scale_factor=scale_factor, shift_factor=shift_factor)
    return FluxAutoencoder(img_shape=(ch_in, resolution, resolution), encoder=encoder, decoder=decoder)


__all__ = ["FluxAutoencoder", "FluxDecoder", "FluxEncoder", "flux_1_autoencoder", "flux_ae_hf_to_tune"]
