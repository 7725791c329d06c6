"""Small training-runtime helpers: profiler set-up, checkpoint path resolution and pruning, vector-quantised embeddings,
layer-slice strings, precision and seed helpers, early-exit loss scales."""
import math

import pytest
import torch
from torch import nn

from torchtune_b200 import training
from torchtune_b200.modules.common_utils import slice_str_to_array
from torchtune_b200.modules.early_exit_loss import inv_l_loss_scale, linear_l_loss_scale, sqrt_l_loss_scale, sum_l_loss_scale, uniform_loss_scale
from torchtune_b200.modules.vq_embeddings import VectorQuantizedEmbeddings
from torchtune_b200.training._profiler import DummyProfiler, setup_torch_profiler
from torchtune_b200.training.checkpointing import _utils as U


def test_disabled_profiler_is_a_no_op_and_enabled_one_fills_schedule_defaults(tmp_path):
    prof, cfg = setup_torch_profiler(enabled=False)
    assert isinstance(prof, DummyProfiler) and cfg["enabled"] is False
    with prof as p:
        p.start(), p.step(), p.stop()

    prof, cfg = setup_torch_profiler(enabled=True, cpu=True, cuda=False, wait_steps=1, active_steps=1, profile_memory=True, output_dir=str(tmp_path / "trace"))
    assert (cfg["wait_steps"], cfg["warmup_steps"], cfg["active_steps"], cfg["num_cycles"]) == (1, 5, 1, 1)  # missing fields take the defaults
    assert cfg["with_stack"] and cfg["record_shapes"]  # memory profiling needs both
    assert (tmp_path / "trace").is_dir()
    assert isinstance(prof, torch.profiler.profile)


def test_checkpoint_path_helpers(tmp_path):
    ckpt, out = tmp_path / "ckpt", tmp_path / "out"
    ckpt.mkdir(), out.mkdir()
    for name in ("model-00001-of-00002.safetensors", "model-00002-of-00002.safetensors"):
        (ckpt / name).write_bytes(b"x")

    files = U.FormattedCheckpointFiles(filename_format="model-{}-of-{}.safetensors", max_filename="00002")
    got = U.get_model_checkpoint_path(files, ckpt, out, should_load_recipe_state=False, has_adapter_checkpoint=False)
    assert [p.name for p in got] == ["model-00001-of-00002.safetensors", "model-00002-of-00002.safetensors"] and all(p.parent == ckpt for p in got)
    with pytest.raises(ValueError):
        U.get_model_checkpoint_path(["missing.safetensors"], ckpt, out, False, False)

    # resuming a full-model run reads what the previous save produced in the output directory
    (out / "model-00001-of-00001.safetensors").write_bytes(b"y")
    got = U.get_model_checkpoint_path(files, ckpt, out, should_load_recipe_state=True, has_adapter_checkpoint=False)
    assert [p.name for p in got] == ["model-00001-of-00001.safetensors"] and got[0].parent == out
    # … unless an adapter is being resumed: the base model still comes from the checkpoint directory
    got = U.get_model_checkpoint_path(files, ckpt, out, should_load_recipe_state=True, has_adapter_checkpoint=True)
    assert all(p.parent == ckpt for p in got)

    assert U.get_recipe_checkpoint_path(out, ckpt, None, should_load_recipe_state=False) is None
    with pytest.raises(ValueError, match="recipe_checkpoint"):
        U.get_recipe_checkpoint_path(out, ckpt, None, should_load_recipe_state=True)
    (ckpt / "recipe_state.pt").write_bytes(b"z")
    assert U.get_recipe_checkpoint_path(out, ckpt, None, should_load_recipe_state=True) == ckpt / "recipe_state.pt"

    assert U.get_adapter_checkpoint_path(out, None, should_load_recipe_state=True) is None
    for n in (0, 2, 10):
        (out / f"epoch_{n}").mkdir()
    (out / "epoch_10" / "adapter_model.pt").write_bytes(b"a")
    assert U.get_largest_iter_folder(out) == "epoch_10"  # numeric, not lexicographic
    assert U.get_adapter_checkpoint_path(out, None, should_load_recipe_state=True) == out / "epoch_10" / "adapter_model.pt"

    with pytest.raises(ValueError):
        U.check_outdir_not_in_ckptdir(ckpt, ckpt / "sub")
    assert U.check_outdir_not_in_ckptdir(ckpt, out)


def test_prune_keeps_the_newest_by_number_and_copy_files_skips_weights(tmp_path):
    dirs = [tmp_path / f"epoch_{n}" for n in (9, 10, 11, 2)]
    for d in dirs:
        d.mkdir()
    U.prune_surplus_checkpoints(dirs, keep_last_n_checkpoints=2)
    assert sorted(p.name for p in tmp_path.iterdir()) == ["epoch_10", "epoch_11"]
    with pytest.raises(ValueError):
        U.prune_surplus_checkpoints(dirs, keep_last_n_checkpoints=0)

    src, dst = tmp_path / "src", tmp_path / "dst"
    (src / "nested").mkdir(parents=True)
    (src / ".git").mkdir()
    (src / "config.json").write_text("{}")
    (src / "nested" / "tokenizer.model").write_text("tok")
    (src / "model.safetensors").write_text("weights")
    (src / ".git" / "HEAD").write_text("ref")
    U.copy_files(src, dst, ignore_suffixes=[".safetensors"])
    assert sorted(str(p.relative_to(dst)) for p in dst.rglob("*") if p.is_file()) == ["config.json", "nested/tokenizer.model"]


def test_safe_torch_load_and_size_parsing(tmp_path):
    path = tmp_path / "w.pt"
    torch.save({"a": torch.arange(6).view(2, 3)}, path)
    assert torch.equal(U.safe_torch_load(path)["a"], torch.arange(6).view(2, 3))
    with pytest.raises(ValueError, match="Unable to load"):
        U.safe_torch_load(tmp_path / "absent.pt")
    assert U.parse_size("5GB") == 5 * 10**9 and U.parse_size(1234) == 1234
    shards = U.shard_state_dict({"a": torch.zeros(100), "b": torch.zeros(100), "c": torch.zeros(10)}, max_shard_size=500)
    assert [sorted(s) for s in shards] == [["a"], ["b", "c"]]


def test_vector_quantised_embeddings_pick_the_nearest_code_and_pass_gradients_through():
    torch.manual_seed(0)
    vq = VectorQuantizedEmbeddings(num_embeddings=7, embedding_dim=5)
    z = torch.randn(2, 3, 5, requires_grad=True)
    q, ids = vq(z)
    nearest = torch.cdist(z.detach().reshape(-1, 5), vq.embedding.detach()).argmin(1).view(2, 3)
    assert torch.equal(ids, nearest)
    assert torch.allclose(q, vq.embedding[ids])
    q.sum().backward()
    assert torch.equal(z.grad, torch.ones_like(z))  # straight-through estimator
    assert torch.equal(vq.decode(ids), vq.embedding[ids])
    with pytest.raises(ValueError):
        vq(torch.randn(1, 2, 4))


def test_layer_slice_strings():
    assert slice_str_to_array("1:3", 5) == [False, True, True, False, False]
    assert slice_str_to_array("::2", 5) == [True, False, True, False, True]
    assert slice_str_to_array("0,4", 5) == [True, False, False, False, True]
    assert slice_str_to_array("2", 4) == [False, False, True, False]
    assert slice_str_to_array(":", 3) == [True, True, True]
    with pytest.raises(AssertionError):
        slice_str_to_array("1,2:3", 5)
    with pytest.raises(AssertionError):
        slice_str_to_array("7", 5)


def test_early_exit_loss_scales():
    """Weights over the layers that carry a loss: a shape in the layer index, early layers scaled by ``e_scale``, the last layer
    never, normalised to one."""
    ids, n = torch.tensor([0.0, 2.0, 3.0]), 4
    assert torch.allclose(uniform_loss_scale(ids, n, e_scale=0.5), torch.tensor([0.25, 0.25, 0.5]))
    assert torch.allclose(linear_l_loss_scale(ids, n, e_scale=0.5), torch.tensor([0.5, 1.5, 4.0]) / 6.0)
    assert torch.allclose(sum_l_loss_scale(ids, n, e_scale=1.0), torch.tensor([1.0, 4.0, 8.0]) / 13.0)
    assert torch.allclose(sqrt_l_loss_scale(ids, n, e_scale=1.0), torch.tensor([1.0, 3.0**0.5, 2.0]) / (3.0 + 3.0**0.5))
    inv = inv_l_loss_scale(ids, n, e_scale=1.0)
    assert inv[0] > inv[1] > inv[2] and float(inv.sum()) == pytest.approx(1.0)
    # without the last layer among them, every entry is an early exit and e_scale cancels in the normalisation
    assert torch.allclose(uniform_loss_scale(torch.tensor([0.0, 1.0]), n, e_scale=0.1), torch.tensor([0.5, 0.5]))


def test_precision_and_seed_helpers():
    assert training.get_dtype("bf16", torch.device("cpu")) is torch.bfloat16 and training.get_dtype("fp32") is torch.float32
    with pytest.raises(ValueError):
        training.get_dtype("int7")
    with training.set_default_dtype(torch.bfloat16):
        assert nn.Linear(2, 2).weight.dtype is torch.bfloat16
    assert nn.Linear(2, 2).weight.dtype is torch.float32
    training.validate_expected_param_dtype(nn.Linear(2, 2).named_parameters(), torch.float32)
    with pytest.raises(ValueError):
        training.validate_expected_param_dtype(nn.Linear(2, 2).named_parameters(), torch.bfloat16)

    assert training.set_seed(123) == 123
    a = torch.rand(3)
    training.set_seed(123)
    assert torch.equal(a, torch.rand(3))
    picked = training.set_seed(None)
    assert isinstance(picked, int) and 0 <= picked < 2**32
    with pytest.raises(ValueError):
        training.set_seed(-1)
    assert math.isfinite(picked)
