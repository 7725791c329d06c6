"""Llama-4 text decoder (mixture of experts, chunked attention, layers without rotary embedding), the CLIP text tower and
Llama-3.2-Vision against the `transformers` implementations on tiny random models, through this package's weight converters.

Two places where the `transformers` port of Llama-3.2-Vision computes something else than this package (and the reference) are
kept out of the comparison, and said here: its vision tower pads every tile's tokens to a multiple of eight and lets real queries
attend to the padded keys (so the tower is composed here from its own sub-modules without the padding), and it does not zero the
cross-attention output of text rows that see no image (so the language model is compared with every row seeing the image; the
behaviour for rows without an image is pinned separately below)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")


def test_llama4_text_decoder_matches_transformers():
    from torchtune_b200.models.llama4 import llama4_decoder
    from torchtune_b200.models.llama4._convert_weights import llama4_hf_to_tune, llama4_tune_to_hf

    torch.manual_seed(0)
    cfg = transformers.Llama4TextConfig(
        vocab_size=128, hidden_size=64, intermediate_size=48, intermediate_size_mlp=96, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16, num_local_experts=4,
        num_experts_per_tok=1, interleave_moe_layer_step=1, max_position_embeddings=64, rms_norm_eps=1e-5, rope_theta=500000.0, rope_scaling=None, no_rope_layers=[1, 1, 1, 0],
        attention_chunk_size=8, use_qk_norm=True, attn_temperature_tuning=False, tie_word_embeddings=False, attn_implementation="eager", pad_token_id=0)
    hf = transformers.Llama4ForCausalLM(cfg).eval().float()
    with torch.no_grad():
        for name, p in hf.named_parameters():
            if "experts" in name or "router" in name:  # these start at zero / uninitialised in a fresh model
                torch.nn.init.normal_(p, std=0.05)
    published = {"language_model." + k: v for k, v in hf.state_dict().items()}
    converted = llama4_hf_to_tune(published)
    mine = llama4_decoder(vocab_size=128, num_layers=4, num_heads=4, num_kv_heads=2, embed_dim=64, hidden_dim=48, max_seq_len=64, rope_base=500000, norm_eps=1e-5, num_experts=4,
                          experts_per_token=1, use_shared_expert=True, use_qk_norm=True, skip_rope_interval=4, attention_chunk_size=8).eval()
    mine.load_state_dict({k[len("decoder."):]: v for k, v in converted.items()})
    tokens = torch.randint(0, 128, (2, 21))  # longer than two attention chunks
    with torch.no_grad():
        want, got = hf(input_ids=tokens).logits, mine(tokens)
    assert torch.allclose(got, want, atol=3e-6), (got - want).abs().max()
    back = llama4_tune_to_hf(converted)
    assert set(back) == set(published) and all(torch.equal(back[k], published[k]) for k in published)


def test_clip_text_encoder_matches_transformers():
    from torchtune_b200.models.clip import clip_text_encoder
    from torchtune_b200.models.clip._convert_weights import clip_text_hf_to_tune

    torch.manual_seed(0)
    cfg = transformers.CLIPTextConfig(vocab_size=100, hidden_size=32, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, max_position_embeddings=16, hidden_act="quick_gelu",
                                      layer_norm_eps=1e-5, eos_token_id=99, pad_token_id=0, bos_token_id=98)
    hf = transformers.CLIPTextModel(cfg).eval()
    mine = clip_text_encoder(embed_dim=32, num_heads=4, num_layers=2, vocab_size=100, max_seq_len=16, norm_eps=1e-5).eval()
    mine.eot_token = 99
    mine.load_state_dict(clip_text_hf_to_tune(hf.state_dict()))
    tokens = torch.randint(1, 97, (3, 16))
    tokens[:, 10], tokens[:, 11:] = 99, 0
    with torch.no_grad():
        want, got = hf(input_ids=tokens).pooler_output, mine(tokens)
    assert torch.allclose(got, want, atol=3e-6), (got - want).abs().max()


_RATIOS = [[1, 1], [1, 2], [1, 3], [1, 4], [2, 1], [2, 2], [3, 1], [4, 1]]


def _mllama():
    from transformers.models.mllama.configuration_mllama import MllamaTextConfig, MllamaVisionConfig

    vision = MllamaVisionConfig(hidden_size=32, num_hidden_layers=4, num_global_layers=2, attention_heads=4, intermediate_size=128, vision_output_dim=96, image_size=16, patch_size=4,
                                max_num_tiles=4, intermediate_layers_indices=[1, 2], supported_aspect_ratios=_RATIOS)
    text = MllamaTextConfig(vocab_size=128, hidden_size=64, num_hidden_layers=5, num_attention_heads=4, num_key_value_heads=2, intermediate_size=96, max_position_embeddings=16384,
                            rope_parameters=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192, rope_theta=500000.0),
                            cross_attention_layers=[3], tie_word_embeddings=False, pad_token_id=0, bos_token_id=1, eos_token_id=2)
    cfg = transformers.MllamaConfig(vision_config=vision, text_config=text, image_token_index=128)
    cfg._attn_implementation = "eager"
    return cfg, transformers.MllamaForConditionalGeneration(cfg).eval().float()


def _native_vision_model():
    from torchtune_b200.models.llama3_2_vision import llama3_2_vision_decoder, llama3_2_vision_encoder
    from torchtune_b200.modules.model_fusion import DeepFusionModel

    enc = llama3_2_vision_encoder(patch_size=4, num_heads=4, clip_embed_dim=32, clip_num_layers=4, clip_hidden_states=[1, 2], num_layers_projection=2, decoder_embed_dim=64, tile_size=16,
                                  max_num_tiles=4, in_channels=3)
    dec = llama3_2_vision_decoder(vocab_size=128, num_layers=4, fusion_interval=4, num_special_tokens=8, num_heads=4, num_kv_heads=2, embed_dim=64, max_seq_len=64, encoder_max_seq_len=68,
                                  rope_base=500000, intermediate_dim=96)
    model = DeepFusionModel(encoder=enc, decoder=dec).eval()
    with torch.no_grad():  # nothing may hide behind a zero gate or an all-ones scale
        for name, p in model.named_parameters():
            if p.numel() == 1:
                torch.nn.init.normal_(p, std=0.5)
            elif "embedding" in name:
                torch.nn.init.normal_(p, std=0.1)
            elif p.ndim >= 2:
                torch.nn.init.normal_(p, std=0.08)
    return model


def _in_memory_key(published: str) -> str:
    """Key of the published checkpoint layout → key of the `transformers` module tree."""
    if published.startswith(("vision_model.", "multi_modal_projector.")):
        return "model." + published
    if published.startswith("language_model.model."):
        return "model.language_model." + published[len("language_model.model."):]
    assert published == "language_model.lm_head.weight", published
    return "lm_head.weight"


def _vision_tower_without_padding(vm, pixel_values, aspect_ratio_ids):
    bsz, nimg, ntile, c, hh, ww = pixel_values.shape
    ids = aspect_ratio_ids.reshape(bsz * nimg, -1)
    x = vm.patch_embedding(pixel_values.reshape(bsz * nimg * ntile, c, hh, ww)).flatten(2).transpose(1, 2)
    _, n, dim = x.shape
    x = vm.pre_tile_positional_embedding(x.reshape(bsz * nimg, ntile, -1, dim), ids)
    x = vm.apply_class_embedding(x.reshape(bsz * nimg * ntile, n, dim))
    n += 1
    x = vm.gated_positional_embedding(x.reshape(bsz * nimg, ntile, n, dim), ids)
    x = vm.layernorm_pre(x).reshape(bsz * nimg, ntile * n, dim)
    taps = []

    def run(layer, h):
        out = layer(h, attention_mask=None)
        return out[0] if isinstance(out, tuple) else out

    for i, layer in enumerate(vm.transformer.layers):
        if i in vm.intermediate_layers_indices:
            taps.append(x)
        x = run(layer, x)
    x = vm.layernorm_post(x)
    x = vm.post_tile_positional_embedding(x.reshape(bsz * nimg, ntile, n, dim), ids).reshape(bsz * nimg, ntile * n, dim)
    for layer in vm.global_transformer.layers:
        x = run(layer, x)
    taps = torch.stack(taps, dim=-1).reshape(bsz, nimg, ntile, n, -1)
    return torch.cat([x.reshape(bsz, nimg, ntile, n, dim), taps], dim=-1)


def test_llama3_2_vision_matches_transformers():
    from transformers.models.mllama.modeling_mllama import _prepare_cross_attention_mask

    from torchtune_b200.models.llama3_2_vision._convert_weights import _vision_args, llama3_vision_hf_to_tune, llama3_vision_tune_to_hf

    torch.manual_seed(0)
    cfg, hf = _mllama()
    mine = _native_vision_model()
    args = _vision_args(cfg.to_dict())
    published = llama3_vision_tune_to_hf(mine.state_dict(), **args)
    hf.load_state_dict({_in_memory_key(k): v for k, v in published.items()})  # strict: the converter covers the whole model

    # and back: everything but the cells of the tile-position grids that no supported aspect ratio reaches
    back = llama3_vision_hf_to_tune(published, **args)
    for key, value in mine.state_dict().items():
        if "tile_pos_embed.embedding" in key or "global_token_positional_embedding" in key:
            reached = torch.zeros(4, 4, dtype=torch.bool)
            for h, w in _RATIOS:
                reached[:h, :w] = True
            assert torch.equal(back[key][reached], value[reached]), key
        else:
            assert torch.equal(back[key], value), key

    bsz, seq = 2, 9
    tokens = torch.randint(3, 120, (bsz, seq))
    tokens[:, 1] = 128  # the image token (first row of the fusion embedding)
    images = torch.randn(bsz, 1, 4, 3, 16, 16)
    for ratio_id, (h, w) in ((6, (2, 2)), (2, (1, 2))):
        tiles = h * w
        img = images.clone()
        img[:, :, tiles:] = 0
        ids = torch.tensor([[ratio_id]] * bsz)
        aspect = torch.tensor([[[h, w]]] * bsz)
        with torch.no_grad():
            states = hf.model.multi_modal_projector(_vision_tower_without_padding(hf.model.vision_model, img, ids)).reshape(bsz, -1, 64)
            got_states = mine.encoder(img, aspect)
        live = tiles * 17
        assert torch.allclose(got_states[:, :live], states[:, :live], atol=1e-5), (got_states[:, :live] - states[:, :live]).abs().max()

        visible = torch.zeros(bsz, seq, 1, 4, dtype=torch.long)
        visible[..., :tiles] = 1
        mask, full_rows = _prepare_cross_attention_mask(visible, num_vision_tokens=17, dtype=torch.float32)
        with torch.no_grad():
            out = hf.model.language_model(input_ids=tokens, cross_attention_states=states, cross_attention_mask=mask, full_text_row_masked_out_mask=full_rows)
            want = hf.lm_head(out.last_hidden_state)
            enc_mask = torch.zeros(bsz, seq, 68, dtype=torch.bool)
            enc_mask[:, :, :live] = True
            got = mine(tokens, encoder_input={"images": img, "aspect_ratio": aspect}, encoder_mask=enc_mask)
        assert torch.allclose(got, want, atol=2e-5), (got - want).abs().max()


def test_text_rows_without_an_image_pass_through_the_fusion_layer():
    mine = _native_vision_model()
    fusion = mine.decoder.layers[3].fusion_layer
    x = torch.randn(2, 5, 64)
    enc = torch.randn(2, 68, 64)
    mask = torch.ones(2, 5, 68, dtype=torch.bool)
    mask[:, :2] = False  # the first two text positions see no image token
    with torch.no_grad():
        out = fusion(x, encoder_input=enc, encoder_mask=mask)
    assert torch.equal(out[:, :2], x[:, :2])
    assert not torch.allclose(out[:, 2:], x[:, 2:])


def test_llama4_early_fusion_matches_transformers():
    """Whole Llama-4 model: the vision tower (2-D rotary embedding per tile, pixel shuffle, adapter MLP), the projector, the image
    tokens scattered into the text sequence, and the mixture-of-experts decoder — through the checkpoint converter in both
    directions."""
    from transformers.models.llama4.configuration_llama4 import Llama4Config, Llama4TextConfig, Llama4VisionConfig

    from torchtune_b200.models.llama4 import llama4_decoder, llama4_vision_encoder
    from torchtune_b200.models.llama4._convert_weights import llama4_hf_to_tune, llama4_tune_to_hf
    from torchtune_b200.modules.model_fusion import EarlyFusionModel

    torch.manual_seed(0)
    vision = Llama4VisionConfig(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128, vision_output_dim=48, image_size=16, patch_size=4, norm_eps=1e-5,
                                pixel_shuffle_ratio=0.5, projector_input_dim=48, projector_output_dim=48, rope_parameters=dict(rope_type="default", rope_theta=10000.0))
    text = Llama4TextConfig(vocab_size=136, hidden_size=64, intermediate_size=48, intermediate_size_mlp=96, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                            num_local_experts=4, num_experts_per_tok=1, interleave_moe_layer_step=1, max_position_embeddings=64, rms_norm_eps=1e-5, rope_theta=500000.0, rope_scaling=None,
                            no_rope_layers=[1, 1, 1, 0], attention_chunk_size=8, use_qk_norm=True, attn_temperature_tuning=False, tie_word_embeddings=False, pad_token_id=0)
    cfg = Llama4Config(vision_config=vision, text_config=text, image_token_index=130, boi_token_index=131, eoi_token_index=132)
    cfg._attn_implementation = "eager"
    hf = transformers.Llama4ForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for name, p in hf.named_parameters():
            if "layernorm" in name.lower() or name.endswith("norm.weight"):
                p.copy_(1.0 + 0.1 * torch.randn_like(p)) if name.endswith("weight") else torch.nn.init.normal_(p, std=0.1)
            else:
                torch.nn.init.normal_(p, std=0.08)

    released = dict(hf.state_dict())  # this model's module tree already has the layout of the released checkpoint
    native = llama4_hf_to_tune(released)
    decoder = llama4_decoder(vocab_size=136, num_layers=4, num_heads=4, num_kv_heads=2, embed_dim=64, hidden_dim=48, max_seq_len=64, rope_base=500000, norm_eps=1e-5, num_experts=4,
                             experts_per_token=1, use_shared_expert=True, use_qk_norm=True, skip_rope_interval=4, attention_chunk_size=8)
    tower = llama4_vision_encoder(patch_size=4, num_heads=4, clip_embed_dim=32, clip_num_layers=2, clip_hidden_states=None, projection_embed_dim=48, decoder_embed_dim=64, tile_size=16,
                                  max_num_tiles=1, in_channels=3)
    mine = EarlyFusionModel(decoder, encoders={"vision": tower}, encoder_tokens={"vision": 130}).eval()
    mine.load_state_dict(native)  # strict

    back = llama4_tune_to_hf(native)
    assert set(back) == set(released) and all(torch.equal(back[k], released[k]) for k in released)

    # two tiles of 4 image tokens each in the first sequence, one in the second
    tokens = torch.randint(3, 128, (2, 19))
    tokens[0, 2:6] = 130
    tokens[0, 9:13] = 130
    tokens[1, 5:9] = 130
    images = torch.randn(3, 3, 16, 16)
    with torch.no_grad():
        want = hf(input_ids=tokens, pixel_values=images).logits
        got = mine(tokens, encoder_input={"vision": {"images": images}})
    assert torch.allclose(got, want, atol=2e-5), (got - want).abs().max()
    with torch.no_grad():
        text_only = torch.randint(3, 128, (2, 19))
        assert torch.allclose(mine(text_only), hf(input_ids=text_only).logits, atol=2e-5)
