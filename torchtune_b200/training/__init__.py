from . import metric_logging
from ._grad_scaler import scale_grads, scale_grads_
from ._model_util import disable_dropout
from .checkpointing import (
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
    Checkpointer,
    CheckpointClient,
    TrainingProgress,
    DistributedCheckpointer,
    FormattedCheckpointFiles,
    FullModelHFCheckpointer,
    FullModelMetaCheckpointer,
    FullModelTorchTuneCheckpointer,
    ModelType,
    update_state_dict_for_classifier,
)
from .lr_schedulers import get_cosine_schedule_with_warmup, get_lr
from .memory import (
    OptimizerInBackwardWrapper,
    apply_selective_activation_checkpointing,
    cleanup_before_training,
    create_optim_in_bwd_wrapper,
    get_memory_stats,
    log_memory_stats,
    register_optim_in_bwd_hooks,
    set_activation_checkpointing,
)
from .pooling import get_unmasked_sequence_lengths
from .precision import get_dtype, set_default_dtype, validate_expected_param_dtype
from .seed import set_seed
from ._activation_offloading import NoOpManager, OffloadActivations, get_act_offloading_ctx_manager
from ._profiler import DEFAULT_PROFILE_DIR, DEFAULT_PROFILER_ACTIVITIES, DEFAULT_SCHEDULE, DEFAULT_TRACE_OPTS, PROFILER_KEY, DummyProfiler, setup_torch_profiler
from ._distributed import (
    VALID_BACKENDS_FOR_MEMORY_STATS,
    LayerwisePreparer,
    ParallelDims,
    gather_cpu_state_dict,
    get_distributed_backend,
    get_context_parallel_manager,
    get_shard_conditions,
    get_train_context,
    prepare_mha_for_tp,
    shard_model,
    get_full_optimizer_state_dict,
    get_world_size_and_rank,
    init_distributed,
    is_distributed,
    load_from_full_model_state_dict,
    load_from_full_optimizer_state_dict,
    materialize,
    set_torch_num_threads,
    validate_no_params_on_meta_device,
)
from . import quantization
from .quantization import convert_to_float8_training, get_quantizer_mode, is_fp8_tensorwise_scaling, swap_lora_linear_with_qat
from ._compile import compile_loss, compile_model
