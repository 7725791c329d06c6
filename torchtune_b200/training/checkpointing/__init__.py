from ._checkpointer import (
    FullModelHFCheckpointer,
    FullModelMetaCheckpointer,
    FullModelTorchTuneCheckpointer,
)
from ._checkpoint_client import CheckpointClient, TrainingProgress
from ._sharded import DistributedCheckpointer
from ._utils import (
    ADAPTER_CONFIG,
    ADAPTER_KEY,
    DATALOADER_KEY,
    EPOCHS_KEY,
    MAX_STEPS_KEY,
    MODEL_KEY,
    OPT_KEY,
    RNG_KEY,
    SEED_KEY,
    STEPS_KEY,
    TOTAL_EPOCHS_KEY,
    VAL_DATALOADER_KEY,
    FormattedCheckpointFiles,
    ModelType,
    get_largest_iter_folder,
    update_state_dict_for_classifier,
)

Checkpointer = FullModelHFCheckpointer

__all__ = [
    "CheckpointClient",
    "TrainingProgress",
    "DistributedCheckpointer",
    "FullModelHFCheckpointer",
    "FullModelMetaCheckpointer",
    "FullModelTorchTuneCheckpointer",
    "ModelType",
    "FormattedCheckpointFiles",
    "update_state_dict_for_classifier",
    "get_largest_iter_folder",
    "ADAPTER_CONFIG",
    "ADAPTER_KEY",
    "EPOCHS_KEY",
    "MAX_STEPS_KEY",
    "MODEL_KEY",
    "OPT_KEY",
    "RNG_KEY",
    "SEED_KEY",
    "STEPS_KEY",
    "TOTAL_EPOCHS_KEY",
    "DATALOADER_KEY",
    "VAL_DATALOADER_KEY",
]
