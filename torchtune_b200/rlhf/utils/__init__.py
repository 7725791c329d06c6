from ._convert_weights import reward_hf_to_tune, reward_tune_to_hf

__all__ = ["reward_hf_to_tune", "reward_tune_to_hf"]
