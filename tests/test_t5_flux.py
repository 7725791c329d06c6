"""T5 encoder against the `transformers` implementation on a tiny random model, and the Flux autoencoder's shapes, sampling and
checkpoint-key conversion."""
import pytest
import torch

from torchtune_b200.models.flux import flux_1_autoencoder
from torchtune_b200.models.flux._convert_weights import ConversionError, flux_ae_hf_to_tune
from torchtune_b200.models.t5 import t5_encoder
from torchtune_b200.models.t5._builders import t5_encoder_hf_to_tune
from torchtune_b200.models.t5._encoder import relative_position_buckets


def _hf_t5():
    transformers = pytest.importorskip("transformers")
    cfg = transformers.T5Config(vocab_size=100, d_model=32, d_kv=8, d_ff=64, num_layers=2, num_heads=4, relative_attention_num_buckets=8,
                                relative_attention_max_distance=16, feed_forward_proj="gated-gelu", layer_norm_epsilon=1e-6, dropout_rate=0.0)
    torch.manual_seed(0)
    return transformers.T5EncoderModel(cfg).eval()


def test_t5_encoder_matches_transformers():
    hf = _hf_t5()
    mine = t5_encoder(embed_dim=32, mlp_dim=64, num_heads=4, head_dim=8, num_layers=2, rel_pos_num_buckets=8, rel_pos_max_dist=16, vocab_size=100,
                      norm_eps=1e-6, max_seq_len=24).eval()
    state = {k: v for k, v in hf.state_dict().items()}
    missing, unexpected = mine.load_state_dict(t5_encoder_hf_to_tune(state), strict=False)
    assert not unexpected and all("bucket" in k or "relative_position" in k for k in missing)
    tokens = torch.randint(0, 100, (3, 24))
    with torch.no_grad():
        want = hf(input_ids=tokens).last_hidden_state
        got = mine(tokens)
    assert torch.allclose(got, want, atol=2e-5), (got - want).abs().max()


def test_t5_relative_position_buckets_are_symmetric_in_sign_and_saturate():
    b = relative_position_buckets(num_buckets=8, max_dist=16, max_seq_len=40)
    assert b.shape[-2:] == (40, 40) and int(b.max()) == 7 and int(b.min()) == 0
    flat = b.reshape(40, 40)
    assert flat[0, 0] == flat[5, 5]  # a function of the offset only
    assert flat[0, 39] == flat[0, 30]  # far keys to the right share the last bucket of their half
    assert flat[39, 0] == flat[39, 9] and flat[39, 0] != flat[0, 39]  # and the two directions use different halves


def test_t5_converter_rejects_unknown_keys():
    with pytest.raises(KeyError):
        t5_encoder_hf_to_tune({"encoder.block.0.layer.0.SelfAttention.bogus": torch.zeros(1)})
    assert t5_encoder_hf_to_tune({"decoder.block.0.x": torch.zeros(1), "shared.weight": torch.zeros(1)}) == {}


def _tiny_ae():
    torch.manual_seed(0)
    return flux_1_autoencoder(resolution=32, ch_base=32, ch_mults=(1, 2), ch_z=4, n_layers_per_resample_block=1, scale_factor=0.5, shift_factor=0.1).eval()


def test_flux_autoencoder_shapes_and_round_trip_of_the_latent_affine():
    ae = _tiny_ae()
    x = torch.randn(2, 3, 32, 32)
    with torch.no_grad():
        z = ae.encode(x)
        y = ae.decode(z)
        y2 = ae(x)
    assert z.shape == (2, 4, 16, 16)  # one downsampling for two channel multipliers
    assert y.shape == x.shape and y2.shape == x.shape
    assert torch.isfinite(y).all()
    # the encoder samples; with the same generator state the result repeats
    torch.manual_seed(3)
    a = ae.encode(x)
    torch.manual_seed(3)
    b = ae.encode(x)
    assert torch.equal(a, b)


def test_flux_autoencoder_trains():
    ae = _tiny_ae().train()
    x = torch.randn(1, 3, 32, 32)
    loss = (ae(x) - x).pow(2).mean()
    loss.backward()
    grads = [p.grad for p in ae.parameters()]
    assert all(g is not None and torch.isfinite(g).all() for g in grads)


def test_flux_checkpoint_keys_convert_onto_the_model():
    torch.manual_seed(0)
    ae = flux_1_autoencoder(resolution=32, ch_base=32, ch_mults=(1, 2, 2, 2), ch_z=4, n_layers_per_resample_block=1)
    native = ae.state_dict()
    # write the native state under the original layout by inverting the documented naming, then convert back
    inv_res = {"main.0": "norm1", "main.2": "conv1", "main.3": "norm2", "main.5": "conv2", "shortcut": "nin_shortcut"}
    inv_attn = {"attn.q_proj": "q", "attn.k_proj": "k", "attn.v_proj": "v", "attn.output_proj": "proj_out", "norm": "norm"}
    n_up = len(ae.decoder.up)
    original = {}
    for key, value in native.items():
        p = key.split(".")
        model = p[0]
        if p[1] == "conv_in":
            new = key
        elif p[1] == "end":
            new = f"{model}.{ {'0': 'norm_out', '2': 'conv_out'}[p[2]] }.{p[3]}"
        elif p[1] == "mid":
            name = {"0": "block_1", "1": "attn_1", "2": "block_2"}[p[2]]
            rest, leaf = ".".join(p[3:-1]), p[-1]
            sub = (inv_attn if p[2] == "1" else inv_res)[rest]
            new = f"{model}.mid.{name}.{sub}.{leaf}"
            if p[2] == "1" and sub != "norm" and leaf == "weight":
                value = value[:, :, None, None]
        elif p[1] in ("down", "up"):
            block = p[2] if p[1] == "down" else str(n_up - 1 - int(p[2]))
            if p[3] == "layers":
                rest, leaf = ".".join(p[5:-1]), p[-1]
                new = f"{model}.{p[1]}.{block}.block.{p[4]}.{inv_res[rest]}.{leaf}"
            else:
                new = ".".join([model, p[1], block] + p[3:])
        else:
            raise AssertionError(key)
        original[new] = value
    assert n_up == 4  # the converter numbers up blocks for the published four-level model
    converted = flux_ae_hf_to_tune(original)
    assert set(converted) == set(native)
    for k in native:
        assert torch.equal(converted[k], native[k])


def test_flux_converter_rejects_unknown_keys():
    with pytest.raises(ConversionError):
        flux_ae_hf_to_tune({"encoder.sideways.0.weight": torch.zeros(1)})
