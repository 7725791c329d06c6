from ._generation import (
    generate,
    generate_next_token,
    get_causal_mask_from_padding_mask,
    get_position_ids_from_padding_mask,
    sample,
)

__all__ = ["generate", "generate_next_token", "get_causal_mask_from_padding_mask", "get_position_ids_from_padding_mask", "sample"]
