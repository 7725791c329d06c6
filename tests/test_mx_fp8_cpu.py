"""Block-scaled (MX) fp8: the CPU oracle of the quantiser and the emulated blockwise training recipe."""
import torch

from torchtune_b200 import training
from torchtune_b200.ops import reference as ref


def test_mx_quantiser_oracle_properties():
    torch.manual_seed(0)
    x = torch.randn(64, 256) * 3
    x[0] = 0
    x[1, 7] = 1000.0
    q, e = ref.mx_quantize(x)
    assert q.shape == x.shape and e.shape == (64, 8) and e.dtype == torch.uint8
    assert q.abs().max() <= 448 and torch.equal(q, q.to(torch.float8_e4m3fn).float())  # values sit on the e4m3 grid
    assert (e[0] == 0).all() and (q[0] == 0).all()  # all-zero blocks
    back = ref.mx_dequantize(q, e)
    blocks, bb = x.reshape(64, 8, 32), back.reshape(64, 8, 32)
    amax = blocks.abs().amax(-1, keepdim=True)
    assert ((blocks - bb).abs() <= amax * 2.0**-3 + 1e-30).all()  # half an e4m3 step of the block's largest binade, with saturation slack
    # the outlier costs precision only inside its own block
    calm = x.clone()
    calm[1, 7] = 0.0
    assert torch.equal(back[1, 32:], ref.mx_roundtrip(calm)[1, 32:]) and abs(back[1, 7] - 1000.0) <= 125  # 1000 / 2 saturates at 448
    # scale exponents are powers of two chosen from the block maximum: amax / 2^e lies in [256, 512)
    scale = torch.ldexp(torch.ones(64, 8), e.int() - 127)
    ratio = (amax.squeeze(-1) / scale)[1:]
    assert ((ratio >= 256) & (ratio < 512)).all()
    # transposed operand: blocks run along the rows of the source
    qt, et = ref.mx_quantize(x, transpose=True)
    assert qt.shape == (256, 64) and et.shape == (256, 2)
    assert torch.equal(qt, ref.mx_quantize(x.t().contiguous())[0])


def test_blockwise_fp8_recipe_swaps_and_trains_on_cpu():
    from torchtune_b200.models.llama2 import llama2

    torch.manual_seed(0)
    model = llama2(vocab_size=64, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=64, max_seq_len=32, intermediate_dim=128)
    plain = [n for n, m in model.named_modules() if isinstance(m, torch.nn.Linear)]
    training.convert_to_float8_training(model, "blockwise")
    swapped = [n for n, m in model.named_modules() if isinstance(m, training.quantization.Float8Linear)]
    assert swapped and "output" not in swapped and len(swapped) == len(plain) - 1
    assert all(m.recipe == "blockwise" for m in model.modules() if isinstance(m, training.quantization.Float8Linear))
    tokens = torch.randint(0, 64, (2, 32))
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    losses = []
    for _ in range(8):
        logits = model(tokens)
        loss = torch.nn.functional.cross_entropy(logits.reshape(-1, 64), tokens.reshape(-1))
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(loss.item())
    assert losses[-1] < losses[0] - 0.3
