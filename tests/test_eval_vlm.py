"""Vision-language evaluation front-end on a tiny deep-fusion model with a stand-in transform: generation runs on the self- and
cross-attention caches and reproduces cache-free greedy decoding; the JSON-lines multimodal task is scored."""
import json

import pytest
import torch
from PIL import Image

from torchtune_b200.evaluation import EvalVLM, evaluate_multimodal_jsonl
from torchtune_b200.models.llama3_2_vision import llama3_2_vision_decoder, llama3_2_vision_encoder
from torchtune_b200.modules.model_fusion import DeepFusionModel

VOCAB, TILES, PATCHES = 100, 4, 17  # 40 × 40 tiles, 10 × 10 patches → 16 patches + class token


class _Tok:
    eos_id, eot_id, pad_id = 1, 2, 0

    def encode(self, text, add_bos=False, add_eos=False):
        return [3 + (ord(c) % 90) for c in text]

    def decode(self, tokens, skip_special_tokens=True):
        return "".join(chr(ord("a") + (t % 26)) for t in tokens)


class _Transform:
    """Messages → tokens, one ``[tiles, 3, 40, 40]`` tensor per image and a cross-attention mask that lets the text after an image
    see that image's tiles."""

    tokenizer, stop_tokens, max_num_tiles, image_seq_len, pad_id = _Tok(), [1, 2], TILES, TILES * PATCHES, 0

    def decode(self, tokens):
        return self.tokenizer.decode(tokens)

    def __call__(self, sample, inference=False):
        tokens, images, masks, starts = [], [], [], []
        for m in sample["messages"]:
            for part in m.content:
                if part["type"] == "image":
                    px = torch.tensor(list(part["content"].resize((40, 40)).getdata()), dtype=torch.float32).view(40, 40, 3).permute(2, 0, 1) / 255.0
                    images.append(px.unsqueeze(0).repeat(2, 1, 1, 1))  # two tiles
                    starts.append(len(tokens))
                    tokens.append(99)  # image token
                else:
                    tokens.extend(self.tokenizer.encode(part["content"]))
        for start, img in zip(starts, images):
            m = torch.zeros(len(tokens), img.shape[0] * PATCHES, dtype=torch.bool)
            m[start:] = True
            masks.append(m)
        return {"tokens": tokens, "encoder_input": {"images": images, "aspect_ratio": [torch.tensor([1, 2])] * len(images)}, "encoder_mask": masks}


def _model():
    torch.manual_seed(0)
    enc = llama3_2_vision_encoder(patch_size=10, num_heads=4, clip_embed_dim=32, clip_num_layers=4, clip_hidden_states=[1, 3], num_layers_projection=2, decoder_embed_dim=48, tile_size=40, max_num_tiles=TILES)
    dec = llama3_2_vision_decoder(vocab_size=VOCAB, num_layers=4, fusion_interval=2, num_special_tokens=8, num_heads=4, num_kv_heads=2, embed_dim=48, max_seq_len=128, encoder_max_seq_len=2 * TILES * PATCHES,
                                  intermediate_dim=96)
    model = DeepFusionModel(decoder=dec, encoder=enc)
    for p in model.parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.2)
    return model.eval()


def test_vlm_generation_on_caches_matches_cache_free_greedy_decoding(tmp_path):
    model, tf = _model(), _Transform()
    lm = EvalVLM(model, tf, device=torch.device("cpu"), dtype=torch.float32, max_seq_length=64, max_images_per_sample=2)
    img = Image.new("RGB", (50, 30), (200, 30, 90))
    got = lm.generate("what is <image> this", [img], max_gen_toks=5)
    assert 1 <= len(got) <= 5

    # oracle: no caches, the whole sequence is recomputed for every new token
    batch = lm.encode_sample("what is <image> this", [img])
    tokens, emask = batch["tokens"], batch["encoder_mask"]
    want = []
    with torch.no_grad():
        for _ in range(len(got)):
            logits = model(tokens, encoder_input=batch["encoder_input"], encoder_mask=emask)[:, -1]
            nxt = int(logits.argmax(-1))
            want.append(nxt)
            tokens = torch.cat([tokens, torch.tensor([[nxt]])], dim=1)
            emask = torch.cat([emask, emask[:, -1:]], dim=1)
    assert got == want

    with pytest.raises(RuntimeError, match="greedy"):
        lm.generate_until([("x <image>", [img], {"temperature": 0.7})])
    assert lm.generate_until([("x <image>", [img], {"max_gen_toks": 3, "until": ["zzzz"]})])[0] == tf.decode(lm.generate("x <image>", [img], 3))

    path = tmp_path / "img.png"
    img.save(path)
    task = tmp_path / "task.jsonl"
    answer = tf.decode(got[:2])
    task.write_text("\n".join(json.dumps(d) for d in [{"query": "what is <image> this", "images": [str(path)], "answer": answer}, {"query": "what is <image> this", "images": [str(path)], "answer": "???"}]))
    res = evaluate_multimodal_jsonl(lm, str(task), max_gen_toks=2)
    assert res == {"exact_match": 0.5, "contains": 0.5, "n": 2}
