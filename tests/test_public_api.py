"""The documented public surface (names a user of the reference imports) resolves in this package."""
import importlib

import pytest

API = {
    "torchtune_b200.config": ["instantiate", "parse", "validate", "log_config"],
    "torchtune_b200.data": [
        "GrammarErrorCorrectionTemplate", "SummarizeTemplate", "QuestionAnswerTemplate", "PromptTemplate", "PromptTemplateInterface", "ChatMLTemplate", "Message", "Role",
        "InputOutputToMessages", "ShareGPTToMessages", "OpenAIToMessages", "ChosenRejectedToMessages", "AlpacaToMessages", "padded_collate", "padded_collate_dpo",
        "padded_collate_packed", "padded_collate_sft", "padded_collate_tiled_images_and_mask", "left_pad_sequence", "validate_messages", "truncate", "load_image",
        "format_content_with_images", "mask_messages",
    ],
    "torchtune_b200.datasets": [
        "alpaca_dataset", "alpaca_cleaned_dataset", "grammar_dataset", "hh_rlhf_helpful_dataset", "samsum_dataset", "slimorca_dataset", "stack_exchange_paired_dataset",
        "cnn_dailymail_articles_dataset", "wikitext_dataset", "instruct_dataset", "chat_dataset", "preference_dataset", "text_completion_dataset", "TextCompletionDataset",
        "ConcatDataset", "PackedDataset", "PreferenceDataset", "SFTDataset",
    ],
    "torchtune_b200.datasets.multimodal": ["llava_instruct_dataset", "the_cauldron_dataset", "vqa_dataset"],
    "torchtune_b200.generation": ["generate", "generate_next_token", "sample", "get_causal_mask_from_padding_mask", "get_position_ids_from_padding_mask"],
    "torchtune_b200.modules": [
        "MultiHeadAttention", "FeedForward", "KVCache", "RotaryPositionalEmbeddings", "RMSNorm", "Fp32LayerNorm", "TanhGate", "TiedLinear", "TransformerSelfAttentionLayer",
        "TransformerCrossAttentionLayer", "TransformerDecoder", "VisionTransformer", "LayerDropout", "prepare_layer_dropout", "classifier_model", "FrozenNF4Linear",
    ],
    "torchtune_b200.modules.loss": ["LinearCrossEntropyLoss", "ForwardKLLoss", "ForwardKLWithChunkedOutputLoss", "ReverseKLWithChunkedOutputLoss", "SymmetricKLWithChunkedOutputLoss"],
    "torchtune_b200.modules.optim": ["OptimizerInBackward"],
    "torchtune_b200.modules.transforms.tokenizers": [
        "SentencePieceBaseTokenizer", "TikTokenBaseTokenizer", "HuggingFaceBaseTokenizer", "ModelTokenizer", "BaseTokenizer", "tokenize_messages_no_special_tokens", "parse_hf_tokenizer_json",
    ],
    "torchtune_b200.modules.peft": [
        "LoRALinear", "DoRALinear", "AdapterModule", "get_adapter_params", "set_trainable_params", "get_adapter_state_dict", "validate_missing_and_unexpected_for_lora", "disable_adapter",
    ],
    "torchtune_b200.modules.model_fusion": ["DeepFusionModel", "EarlyFusionModel", "FusionLayer", "FusionEmbedding", "register_fusion_module", "get_fusion_params"],
    "torchtune_b200.modules.common_utils": ["reparametrize_as_dtype_state_dict_post_hook", "local_kv_cache", "disable_kv_cache", "delete_kv_caches"],
    "torchtune_b200.modules.embedding_utils": ["resize_token_embeddings"],
    "torchtune_b200.modules.transforms": ["Transform", "VisionCrossAttentionMask"],
    "torchtune_b200.modules.moe": ["MoE", "GroupedExperts", "LoRAGroupedExperts", "TokenChoiceTopKRouter"],
    "torchtune_b200.rlhf": ["estimate_advantages", "get_rewards_ppo", "truncate_sequence_at_first_stop_token"],
    "torchtune_b200.rlhf.loss": ["PPOLoss", "DPOLoss", "RSOLoss"],
    "torchtune_b200.training": [
        "FullModelHFCheckpointer", "FullModelMetaCheckpointer", "FullModelTorchTuneCheckpointer", "ModelType", "FormattedCheckpointFiles", "update_state_dict_for_classifier",
        "get_dtype", "set_default_dtype", "validate_expected_param_dtype", "get_quantizer_mode", "init_distributed", "is_distributed", "gather_cpu_state_dict",
        "get_distributed_backend", "apply_selective_activation_checkpointing", "set_activation_checkpointing", "OptimizerInBackwardWrapper", "create_optim_in_bwd_wrapper",
        "register_optim_in_bwd_hooks", "get_cosine_schedule_with_warmup", "get_lr", "get_memory_stats", "log_memory_stats", "setup_torch_profiler",
        "get_unmasked_sequence_lengths", "disable_dropout", "set_seed",
    ],
    "torchtune_b200.training.metric_logging": ["CometLogger", "WandBLogger", "TensorBoardLogger", "StdoutLogger", "DiskLogger", "MLFlowLogger"],
    "torchtune_b200.utils": ["batch_to_device", "get_device", "get_logger", "torch_version_ge", "get_world_size_and_rank"],
}

MODEL_BUILDERS = {
    "llama2": ["llama2_7b", "llama2_13b", "llama2_70b", "lora_llama2_7b", "qlora_llama2_7b", "llama2_tokenizer"],
    "llama3": ["llama3_8b", "llama3_70b", "lora_llama3_8b", "qlora_llama3_8b", "llama3_tokenizer"],
    "llama3_1": ["llama3_1_8b", "llama3_1_70b", "llama3_1_405b", "lora_llama3_1_8b", "qlora_llama3_1_8b"],
    "llama3_2": ["llama3_2_1b", "llama3_2_3b", "lora_llama3_2_1b", "qlora_llama3_2_3b"],
    "llama3_2_vision": ["llama3_2_vision_11b", "lora_llama3_2_vision_11b", "llama3_2_vision_transform"],
    "llama3_3": ["llama3_3_70b", "lora_llama3_3_70b"],
    "llama4": ["llama4_scout_17b_16e", "llama4_maverick_17b_128e", "lora_llama4_scout_17b_16e", "llama4_transform"],
    "mistral": ["mistral_7b", "lora_mistral_7b", "qlora_mistral_7b", "mistral_tokenizer"],
    "gemma": ["gemma_2b", "gemma_7b", "lora_gemma_2b", "gemma_tokenizer"],
    "gemma2": ["gemma2_2b", "gemma2_9b", "gemma2_27b", "lora_gemma2_2b"],
    "phi3": ["phi3_mini", "lora_phi3_mini", "phi3_mini_tokenizer"],
    "phi4": ["phi4_14b", "lora_phi4_14b", "phi4_tokenizer"],
    "qwen2": ["qwen2_0_5b", "qwen2_1_5b", "qwen2_7b", "lora_qwen2_7b", "qwen2_tokenizer"],
    "qwen2_5": ["qwen2_5_0_5b", "qwen2_5_7b_instruct", "qwen2_5_72b_instruct", "lora_qwen2_5_7b_instruct", "qwen2_5_tokenizer"],
    "qwen3": ["qwen3_0_6b_base", "qwen3_8b_instruct", "qwen3_32b", "lora_qwen3_8b_instruct", "qwen3_tokenizer"],
    "clip": ["clip_vision_encoder", "clip_text_encoder", "CLIPImageTransform"],
}


@pytest.mark.parametrize("module", sorted(API))
def test_documented_names_resolve(module):
    mod = importlib.import_module(module)
    missing = [n for n in API[module] if not hasattr(mod, n)]
    assert not missing, f"{module} lacks {missing}"


@pytest.mark.parametrize("family", sorted(MODEL_BUILDERS))
def test_model_builders_resolve(family):
    mod = importlib.import_module(f"torchtune_b200.models.{family}")
    missing = [n for n in MODEL_BUILDERS[family] if not hasattr(mod, n)]
    assert not missing, f"models.{family} lacks {missing}"


def test_recipe_facing_sharding_and_mask_helpers():
    """Names that user recipes import from ``training`` / ``modules`` / ``modules.peft`` and what they do here."""
    import contextlib

    import torch

    from torchtune_b200 import training
    from torchtune_b200.models.llama3_1 import llama3_1
    from torchtune_b200.modules import create_block_causal_mask, packed_block_causal_mask
    from torchtune_b200.modules.peft import TrainableParams
    from torchtune_b200.parallel.cp import ContextParallelContext
    from torchtune_b200.training.checkpointing import get_largest_iter_folder  # noqa: F401

    for name in ("DEFAULT_PROFILE_DIR", "DEFAULT_PROFILER_ACTIVITIES", "DEFAULT_SCHEDULE", "DEFAULT_TRACE_OPTS", "PROFILER_KEY"):
        assert hasattr(training, name)
    assert [p.value for p in TrainableParams] == ["full", "lora", "frozen"]

    lens = [torch.tensor([2, 3]), torch.tensor([4, 1])]
    dense = create_block_causal_mask(lens)
    assert dense.shape == (2, 5, 5) and dense[0, 1].tolist() == [True, True, False, False, False] and dense[0, 4].tolist() == [False, False, True, True, True]
    packed = packed_block_causal_mask(lens)
    assert packed.causal and packed.doc_ids.tolist() == [[0, 0, 1, 1, 1], [0, 0, 0, 0, 1]]

    assert training.get_shard_conditions("decoder.layers.3", None) and not training.get_shard_conditions("layers.3.attn", None)
    assert training.get_shard_conditions("output", None, ["output"])

    arch = dict(vocab_size=64, num_layers=1, num_heads=4, num_kv_heads=2, embed_dim=32, max_seq_len=32, intermediate_dim=48)
    model = training.prepare_mha_for_tp(llama3_1(**arch), 2)
    attn = model.layers[0].attn
    assert (attn.num_heads, attn.num_kv_heads, attn.embed_dim) == (2, 1, 16)

    x = torch.arange(16).view(2, 8)
    cp = ContextParallelContext(None, world=2, rank=1)
    with training.get_context_parallel_manager(enabled=True, cp=cp)([x]):
        assert x.tolist() == [[4, 5, 6, 7], [12, 13, 14, 15]]
    assert x.shape == (2, 8) and x[1, 0] == 8
    with training.get_context_parallel_manager(enabled=False)([x]):
        assert x.shape == (2, 8)
    assert isinstance(training.get_train_context(True)(), contextlib.nullcontext)

    sharded = training.shard_model(llama3_1(**arch), min_numel=1)  # one process: every shard is the whole weight
    assert type(sharded.layers[0].attn.q_proj).__name__ == "ShardedLinear"
    tokens = torch.randint(0, 64, (2, 8))
    assert sharded(tokens).shape == (2, 8, 64)


def test_tensor_parallel_plan_components_describe_the_built_in_layout():
    import pytest

    from torchtune_b200.models.llama3 import base_llama_tp_plan
    from torchtune_b200.models.llama3._parallelism import validate_tp_plan
    from torchtune_b200.models.llama4 import decoder_only_tp_plan

    plan = base_llama_tp_plan()
    assert plan["layers.*.attn.q_proj"] == "column_parallel" and plan["layers.*.mlp.w2"] == "row_parallel" and plan["norm"] == "sequence_parallel"
    validate_tp_plan(plan)
    validate_tp_plan(base_llama_tp_plan(enable_fp8_training=True))
    validate_tp_plan(decoder_only_tp_plan())
    with pytest.raises(ValueError, match="implements"):
        validate_tp_plan({"layers.*.mlp.w2": "column_parallel"})
    with pytest.raises(ValueError, match="does not shard"):
        validate_tp_plan({"layers.*.attn.pos_embeddings": "row_parallel"})
