"""MoE, vision transformer, model fusion, Llama 3.2 Vision and Llama 4 on CPU against dense /
loop oracles written directly in torch."""
import torch
import torch.nn.functional as F

from torchtune_b200.models.clip import CLIPImageTransform, CLIPTokenizer, clip_text_encoder, clip_vision_encoder
from torchtune_b200.models.llama3_2_vision import llama3_2_vision_decoder, llama3_2_vision_encoder, llama3_vision_hf_to_tune, llama3_vision_tune_to_hf
from torchtune_b200.models.llama4 import Llama4Tokenizer, get_chunked_attention_mask, llama4_decoder, llama4_hf_to_tune, llama4_tune_to_hf, llama4_vision_encoder
from torchtune_b200.modules import Linear
from torchtune_b200.modules.model_fusion import DeepFusionModel, EarlyFusionModel, FusionEmbedding, FusionLayer, get_fusion_params, register_fusion_module
from torchtune_b200.modules.moe import GroupedExperts, LoRAGroupedExperts, MoE, TokenChoiceTopKRouter, generate_permute_indices
from torchtune_b200.modules.moe.indices import fill_indices_cpu
from torchtune_b200.modules.transforms.vision_utils import find_supported_resolutions, get_canvas_best_fit, get_inscribed_size, pad_dim_to_size, resize_with_pad, tile_crop
from torchtune_b200.ops.mask import AttentionMask


def test_moe_matches_per_token_oracle_and_backprops():
    torch.manual_seed(0)
    E, k, dim, hid = 4, 2, 16, 32
    experts = GroupedExperts(dim=dim, hidden_dim=hid, num_experts=E)
    router = TokenChoiceTopKRouter(gate=Linear(dim, E, bias=False), dim=dim, num_experts=E, experts_per_token=k)
    shared = torch.nn.Linear(dim, dim, bias=False)
    moe = MoE(experts=experts, router=router, shared_expert=shared)
    x = torch.randn(2, 5, dim, requires_grad=True)
    y = moe(x)
    flat = x.reshape(-1, dim)
    scores, idx = torch.sigmoid(router.gate(flat)).topk(k, 1)
    want = shared(flat).clone()
    for t in range(flat.shape[0]):
        for j in range(k):
            e = idx[t, j]
            xi = flat[t] * scores[t, j]
            want[t] = want[t] + (F.silu(xi @ experts.gate_proj[e]) * (xi @ experts.up_proj[e])) @ experts.down_proj[e]
    torch.testing.assert_close(y.reshape(-1, dim), want, rtol=1e-4, atol=1e-5)
    y.sum().backward()
    assert x.grad is not None and experts.gate_proj.grad is not None and router.gate.weight.grad is not None


def test_lora_experts_start_equal_to_base_and_declare_adapters():
    torch.manual_seed(0)
    base = GroupedExperts(dim=8, hidden_dim=16, num_experts=3)
    lora = LoRAGroupedExperts(dim=8, hidden_dim=16, rank=2, alpha=4.0, num_experts=3)
    with torch.no_grad():
        for n in ("gate_proj", "up_proj", "down_proj"):
            getattr(lora, n).copy_(getattr(base, n))
    x = torch.randn(7, 8)
    counts = torch.tensor([3, 0, 4])
    torch.testing.assert_close(lora(x, counts), base(x, counts))
    assert set(lora.adapter_params()) == {"lora_gate_a", "lora_gate_b", "lora_up_a", "lora_up_b", "lora_down_a", "lora_down_b"}


def test_permute_indices_match_loop_oracle():
    g = torch.Generator().manual_seed(1)
    for ranks, experts, align in ((2, 4, 8), (4, 2, 16), (1, 3, 4)):
        counts = torch.randint(0, 9, (ranks * experts,), generator=g)
        perm, sizes, offsets = generate_permute_indices(counts, experts, ranks, 256, align)
        start = counts.cumsum(0) - counts
        want = fill_indices_cpu(counts, start, offsets - sizes, experts, ranks, 256)
        assert torch.equal(perm, want)
        from torchtune_b200.modules.moe.indices import fill_indices_wrapper

        assert torch.equal(fill_indices_wrapper(counts, start, offsets - sizes, experts, ranks, 256), want)
        assert (sizes % align == 0).all() and (sizes >= counts.view(ranks, experts).sum(0)).all()


def test_vision_utils():
    res = find_supported_resolutions(4, 10)
    assert set(res) == {(10, 10), (10, 20), (20, 10), (10, 30), (30, 10), (10, 40), (40, 10), (20, 20)}
    img = torch.rand(3, 25, 12)
    assert get_canvas_best_fit(img, torch.tensor(res), resize_to_max_canvas=False) == (30, 10) or get_canvas_best_fit(img, torch.tensor(res), False)[0] >= 20
    assert get_inscribed_size((200, 100), (100, 100), None) == (100, 50)
    out = resize_with_pad(img, (40, 20), "bilinear", max_size=None)
    assert out.shape == (3, 40, 20) and (out[:, :, 19:] == 0).all()  # 25x12 → 40x19, padded on the right
    tiles = tile_crop(torch.arange(3 * 4 * 6).float().reshape(3, 4, 6), 2)
    assert tiles.shape == (6, 3, 2, 2) and tiles[1, 0, 0, 0] == 2 and tiles[3, 0, 0, 0] == 12
    assert pad_dim_to_size(torch.ones(2, 3), 5, dim=0).shape == (5, 3)


def test_patch_embedding_equals_conv_and_vit_shapes():
    torch.manual_seed(0)
    enc = clip_vision_encoder(tile_size=40, patch_size=10, embed_dim=32, num_layers=3, num_heads=4, out_indices=[1, 3], max_num_tiles=4)
    conv = torch.nn.Conv2d(3, 32, 10, 10, bias=False)
    conv.weight.data.copy_(enc.conv.weight.data)
    x = torch.randn(2, 3, 40, 40)
    torch.testing.assert_close(enc.conv(x), conv(x).flatten(2).transpose(1, 2), rtol=1e-4, atol=1e-5)
    sample = CLIPImageTransform(tile_size=40, max_num_tiles=4, dtype=torch.float32, image_mean=[0.5] * 3, image_std=[0.2] * 3)({"image": torch.randint(0, 255, (3, 70, 30), dtype=torch.uint8)})
    assert sample["image"].shape == (2, 3, 40, 40) and sample["aspect_ratio"].tolist() == [2, 1]
    tokens, hidden = enc(sample["image"][None, None], sample["aspect_ratio"][None, None])
    assert tokens.shape == (1, 1, 2, 17, 32) and len(hidden) == 2
    # a checkpoint trained with 4 tiles loads into a 2-tile model (position tables are interpolated)
    small = clip_vision_encoder(tile_size=40, patch_size=10, embed_dim=32, num_layers=3, num_heads=4, max_num_tiles=2)
    small.load_state_dict(enc.state_dict())
    assert small.token_pos_embedding.global_token_positional_embedding.shape == (2, 2, 17, 32)


def test_clip_text_encoder_and_tokenizer(tmp_path):
    merges = tmp_path / "merges.txt"
    merges.write_text("#version: 0.2\nh e\nl l\nhe ll\nhell o</w>\nw o\n")
    tok = CLIPTokenizer(str(merges), max_seq_len=8)
    ids = tok.encode("Hello wo")
    assert ids[0] == tok.sot_token and ids[-1] == tok.eot_token
    assert tok.encoder["hello</w>"] in ids
    assert tok.decode(ids[1:-1]).strip() == "hello wo"
    assert len(tok.encode("hello " * 20)) == 8
    enc = clip_text_encoder(embed_dim=32, num_heads=4, num_layers=2, vocab_size=tok.eot_token + 1, max_seq_len=8)
    enc.eot_token = tok.eot_token
    assert enc(torch.tensor([ids])).shape == (1, 32)


def test_fusion_layer_and_embedding_state_dict_layout():
    layer = torch.nn.Linear(4, 4)
    fusion = torch.nn.Linear(4, 4)
    fl = FusionLayer(layer, fusion)
    sd = fl.state_dict()
    assert set(sd) == {"weight", "bias", "fusion_layer.weight", "fusion_layer.bias"}
    fl2 = FusionLayer(torch.nn.Linear(4, 4), torch.nn.Linear(4, 4))
    fl2.load_state_dict(sd)
    assert torch.equal(fl2.layer.weight, layer.weight)
    assert fl.fusion_params() == ["fusion_layer.weight", "fusion_layer.bias"]
    emb = FusionEmbedding(10, 3, 6)
    assert set(emb.state_dict()) == {"weight", "fusion_embedding.weight"}
    out = emb(torch.tensor([[0, 9, 10, 12]]))
    assert torch.equal(out[0, 1], emb.embedding.weight[9]) and torch.equal(out[0, 3], emb.fusion_embedding.weight[2])
    register_fusion_module(fusion)
    assert set(get_fusion_params(torch.nn.ModuleDict({"a": fusion}))) == {"a.weight", "a.bias"}


def _tiny_vision_model():
    enc = llama3_2_vision_encoder(patch_size=10, num_heads=4, clip_embed_dim=32, clip_num_layers=4, clip_hidden_states=[1, 3], num_layers_projection=2, decoder_embed_dim=48, tile_size=40, max_num_tiles=4)
    dec = llama3_2_vision_decoder(vocab_size=100, num_layers=4, fusion_interval=2, num_special_tokens=8, num_heads=4, num_kv_heads=2, embed_dim=48, max_seq_len=64, encoder_max_seq_len=200, intermediate_dim=96)
    return DeepFusionModel(decoder=dec, encoder=enc, decoder_trainable=False, encoder_trainable=True, fusion_trainable=True)


def test_llama3_2_vision_forward_trainability_and_hf_round_trip():
    torch.manual_seed(0)
    model = _tiny_vision_model()
    names = {n for n, p in model.named_parameters() if p.requires_grad}
    assert any("fusion_layer" in n for n in names) and any(n.startswith("encoder.clip") for n in names)
    assert not any(n.startswith("decoder.layers.0.attn") for n in names)
    tokens = torch.randint(0, 108, (2, 12))
    images = torch.randn(2, 1, 4, 3, 40, 40)
    ar = torch.tensor([[[2, 2]], [[1, 2]]])
    emask = torch.ones(2, 12, 4 * 17, dtype=torch.bool)
    emask[0, :3] = False  # first tokens precede the image: they must ignore it entirely
    out = model(tokens, encoder_input={"images": images, "aspect_ratio": ar}, encoder_mask=emask)
    assert out.shape == (2, 12, 100) and out.isfinite().all()
    out.sum().backward()
    ratios = [(1, 1), (1, 2), (1, 3), (1, 4), (2, 1), (2, 2), (3, 1), (4, 1)]
    args = dict(num_heads=4, num_kv_heads=2, dim=48, vocab_size=100, cross_attention_layers=[1, 4], encoder_dim=32, tile_size=40, num_tiles=4, supported_aspect_ratios=ratios)
    sd = model.state_dict()
    hf = llama3_vision_tune_to_hf(sd, **args)
    assert hf["language_model.model.embed_tokens.weight"].shape == (108, 48)
    assert "language_model.model.layers.1.cross_attn.q_proj.weight" in hf and "language_model.model.layers.2.self_attn.q_proj.weight" in hf
    back = llama3_vision_hf_to_tune(hf, **args)
    assert set(back) == set(sd)
    for k in sd:
        if k.endswith("tile_pos_embed.embedding") or k.endswith("global_token_positional_embedding"):
            for h, w in ratios:  # only grid cells reachable by a supported aspect ratio survive the HF layout
                if h * w == 4:
                    assert torch.equal(back[k][:h, :w], sd[k][:h, :w])
        else:
            assert torch.equal(back[k], sd[k]), k


def test_llama4_layers_masks_and_round_trip():
    torch.manual_seed(0)
    dec = llama4_decoder(vocab_size=120, num_layers=4, num_heads=4, num_kv_heads=2, embed_dim=32, hidden_dim=48, max_seq_len=64, num_experts=4, skip_rope_interval=2, attention_chunk_size=8,
                         use_scaled_rope=True, moe_every_n_layers=2, mlp_hidden_dim=64)
    assert [type(l.mlp).__name__ for l in dec.layers] == ["FeedForward", "MoE", "FeedForward", "MoE"]
    assert [l.attn.pos_embeddings is not None for l in dec.layers] == [True, False, True, False]
    enc = llama4_vision_encoder(patch_size=5, num_heads=4, clip_embed_dim=16, clip_num_layers=2, projection_embed_dim=24, decoder_embed_dim=32, tile_size=20, max_num_tiles=4)
    model = EarlyFusionModel(dec, encoders={"vision": enc}, encoder_tokens={"vision": 119}, decoder_trainable=True, encoders_trainable=False, fusion_trainable=True)
    tokens = torch.randint(0, 118, (2, 20))
    tokens[0, 2:6] = 119
    tokens[1, 5:9] = 119
    images = torch.randn(2, 3, 20, 20)
    out = model(tokens, encoder_input={"vision": {"images": images}})
    assert out.shape == (2, 20, 120) and out.isfinite().all()
    # the spliced positions really carry the projected vision tokens
    vis = enc(images).reshape(-1, 32)
    emb = model.decoder.tok_embeddings(torch.where(tokens == 119, torch.zeros_like(tokens), tokens)).masked_scatter((tokens == 119).unsqueeze(-1), vis)
    torch.testing.assert_close(model.decoder(tokens=None, input_embeds=emb), out)
    sd = model.state_dict()
    hf = llama4_tune_to_hf(sd)
    assert hf["language_model.model.layers.1.feed_forward.experts.gate_up_proj"].shape == (4, 32, 96)
    assert hf["vision_model.patch_embedding.linear.weight"].shape == (16, 75)
    back = llama4_hf_to_tune(hf)
    assert set(back) == set(sd) and all(torch.equal(sd[k], back[k]) for k in sd)


def test_chunked_attention_mask():
    m = get_chunked_attention_mask(None, 4, 1, 8)
    assert isinstance(m, AttentionMask) and m.chunk == 4 and m.causal
    dense = get_chunked_attention_mask(torch.ones(1, 8, 8, dtype=torch.bool).tril(), 4, 1, 8)
    assert dense[0, 5].tolist() == [False] * 4 + [True, True, False, False]


def test_llama4_tokenizer_image_grid(tmp_path):
    from tokenizer_assets import write_tiktoken_file

    path = write_tiktoken_file(tmp_path / "tok.model")
    special = {k: 300 + i for i, k in enumerate(k for k in __import__("torchtune_b200").models.llama4._tokenizer.SPECIAL_TOKENS if "_reserved_special_token_" not in k)}
    tok = Llama4Tokenizer(str(path), special_tokens=special)
    one = tok._image_tokens(3, torch.tensor([1, 1]))
    assert one == [tok.image_start, tok.image_id, tok.patch_id, tok.patch_id, tok.patch_id, tok.image_end]
    grid = tok._image_tokens(1, torch.tensor([2, 2]))
    assert grid == [tok.image_start, tok.patch_id, tok.tile_x_separator, tok.patch_id, tok.tile_y_separator, tok.patch_id, tok.tile_x_separator, tok.patch_id, tok.tile_y_separator, tok.image_id, tok.patch_id, tok.image_end]


def test_export_modules_match_training_modules():
    from torchtune_b200.models.llama2 import llama2
    from torchtune_b200.modules._export import replace_mha_with_inference_mha, replace_tile_positional_embedding, replace_tiled_token_positional_embedding

    torch.manual_seed(0)
    model = llama2(vocab_size=64, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=32, max_seq_len=32, intermediate_dim=48).eval()
    tokens = torch.randint(0, 64, (2, 9))
    want = model(tokens)
    keys = set(model.state_dict())
    replace_mha_with_inference_mha(model)
    assert set(model.state_dict()) == keys
    torch.testing.assert_close(model(tokens), want, rtol=1e-5, atol=1e-5)
    exported = torch.export.export(model.layers[0].attn, (torch.randn(2, 9, 32), torch.randn(2, 9, 32)))
    assert exported is not None

    enc = clip_vision_encoder(tile_size=40, patch_size=10, embed_dim=32, num_layers=1, num_heads=4, max_num_tiles=4).eval()
    with torch.no_grad():
        enc.token_pos_embedding.gate.fill_(0.7)
        enc.pre_tile_pos_embed.gate.fill_(0.3)
        enc.post_tile_pos_embed.gate.fill_(-0.4)
    images = torch.randn(2, 1, 4, 3, 40, 40)
    ar = torch.tensor([[[2, 2]], [[1, 3]]])
    want, _ = enc(images, ar)
    replace_tile_positional_embedding(enc)
    replace_tiled_token_positional_embedding(enc)
    got, _ = enc(images, ar)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)


def test_lora_llama4_vision_encoder_builders():
    """Adapters on the CLIP tower and / or the projection head: zero-initialised B matrices leave the output equal to the plain
    encoder with the same base weights; the switches choose where adapters are attached."""
    import torch

    from torchtune_b200.models.llama4 import llama4_vision_encoder, lora_llama4_vision_encoder
    from torchtune_b200.modules.peft import get_adapter_params

    kw = dict(patch_size=14, num_heads=4, clip_embed_dim=64, clip_num_layers=2, projection_embed_dim=96, decoder_embed_dim=48, tile_size=56, max_num_tiles=1)
    torch.manual_seed(0)
    plain = llama4_vision_encoder(**kw)
    lora = lora_llama4_vision_encoder(True, True, ["q_proj", "v_proj"], apply_lora_to_mlp=True, apply_lora_to_output=True, lora_rank=4, lora_alpha=8, **kw)
    adapters = get_adapter_params(lora)
    assert any(k.startswith("clip.") for k in adapters) and any(k.startswith("projection.") for k in adapters)
    missing, unexpected = lora.load_state_dict(plain.state_dict(), strict=False)
    assert not unexpected and all("lora_" in k for k in missing)
    x = torch.randn(3, 3, 56, 56)
    torch.testing.assert_close(lora(x), plain(x), rtol=1e-5, atol=1e-5)
    head_only = lora_llama4_vision_encoder(False, True, ["q_proj"], apply_lora_to_output=True, lora_rank=4, lora_alpha=8, **kw)
    assert all(k.startswith("projection.") for k in get_adapter_params(head_only)) and len(get_adapter_params(head_only)) == 6
    assert len(get_adapter_params(lora_llama4_vision_encoder(False, True, ["q_proj"], apply_lora_to_output=False, lora_rank=4, lora_alpha=8, **kw))) == 0


def test_whole_decoder_exports_with_and_without_kv_cache():
    """``torch.export`` of the complete decoder after the export-friendly attention swap: the exported program reproduces eager
    logits, and — with KV caches set up — a prefill followed by single-token steps through the *exported* module (whose cache
    buffers are graph state) reproduces the cache-free forward pass."""
    from torchtune_b200.models.llama2 import llama2
    from torchtune_b200.modules._export import replace_mha_with_inference_mha

    torch.manual_seed(0)
    model = llama2(vocab_size=64, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=32, max_seq_len=32, intermediate_dim=48).eval()
    replace_mha_with_inference_mha(model)
    tokens = torch.randint(0, 64, (2, 9))
    with torch.no_grad():
        want = model(tokens)
        program = torch.export.export(model, (tokens,))
        torch.testing.assert_close(program.module()(tokens), want, rtol=1e-5, atol=1e-5)

        model.setup_caches(batch_size=2, dtype=torch.float32, decoder_max_seq_len=12)
        causal = torch.tril(torch.ones(12, 12, dtype=torch.bool))
        pos = torch.arange(12)
        prefill_kwargs = {"mask": causal[None, :5].expand(2, -1, -1), "input_pos": pos[None, :5].expand(2, -1)}
        step_kwargs = {"mask": causal[None, 5:6].expand(2, -1, -1), "input_pos": pos[None, 5:6].expand(2, -1)}
        prefill = torch.export.export(model, (tokens[:, :5],), prefill_kwargs).module()
        step = torch.export.export(model, (tokens[:, 5:6],), step_kwargs).module()
        # the two exported programs own separate copies of the cache buffers: carry the state over explicitly
        out = [prefill(tokens[:, :5], **prefill_kwargs)]
        step.load_state_dict(prefill.state_dict(), strict=False)
        for name, buf in prefill.named_buffers():
            dict(step.named_buffers())[name].copy_(buf)
        for t in range(5, 9):
            out.append(step(tokens[:, t : t + 1], mask=causal[None, t : t + 1].expand(2, -1, -1), input_pos=pos[None, t : t + 1].expand(2, -1)))
        torch.testing.assert_close(torch.cat(out, dim=1), want, rtol=1e-4, atol=1e-4)
