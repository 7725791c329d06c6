from .dpo import DPOLoss, PreferenceLoss, RSOLoss
from .ppo import PPOLoss

__all__ = ["DPOLoss", "RSOLoss", "PPOLoss", "PreferenceLoss"]
