import argparse

import pytest
import torch

from torchtune_b200 import config
from torchtune_b200.config import ConfigError, DictConfig, InstantiationError, ListConfig, OmegaConf
from torchtune_b200.config._utils import _merge_yaml_and_cli_args


def test_access_styles_and_interpolation():
    cfg = OmegaConf.create({"a": 1, "out": "/tmp/x", "b": {"c": "${a}", "p": "${out}/logs"}, "l": [1, {"k": "${b.c}"}]})
    assert cfg.a == cfg["a"] == 1
    assert cfg.b.c == 1 and cfg.b.p == "/tmp/x/logs"
    assert cfg.get("missing") is None and cfg.get("missing", 5) == 5
    assert "a" in cfg and "zz" not in cfg
    assert isinstance(cfg.l, ListConfig) and cfg.l[1].k == 1
    assert cfg.pop("a") == 1 and "a" not in cfg
    with pytest.raises(AttributeError):
        cfg.nope
    assert OmegaConf.to_container(cfg.b, resolve=False)["c"] == "${a}"


def test_yaml_scientific_floats_and_dotlist():
    cfg = OmegaConf.create("lr: 2e-5\neps: 1.0e-8\n")
    assert isinstance(cfg.lr, float) and cfg.lr == 2e-5
    d = OmegaConf.from_dotlist(["a.b=3", "c=[1,2]", "d='json'", "e=x.y.Z"])
    assert d.a.b == 3 and list(d.c) == [1, 2] and d.d == "json" and d.e == "x.y.Z"


def test_merge_cli_overrides_component_and_remove():
    ns = argparse.Namespace(a=1, b={"_component_": "torch.nn.Linear", "in_features": 2, "out_features": 3}, c={"d": 4, "e": 5}, f={"max_filename": "00001"})
    out = _merge_yaml_and_cli_args(ns, ["b=torch.nn.Bilinear", "b.out_features=7", "~c.d", "a=None", "f.max_filename=00004"])
    assert out.b._component_ == "torch.nn.Bilinear" and out.b.out_features == 7
    assert "d" not in out.c and out.c.e == 5
    assert out.a is None
    assert out.f.max_filename == "00004"
    with pytest.raises(ValueError):
        _merge_yaml_and_cli_args(argparse.Namespace(b={"_component_": "x"}), ["~b"])
    with pytest.raises(ValueError):
        _merge_yaml_and_cli_args(argparse.Namespace(a=1), ["novalue"])


class Spice:
    def __init__(self, heat):
        self.heat = heat


class Food:
    def __init__(self, seed, ingredient, extras=None):
        self.seed, self.ingredient, self.extras = seed, ingredient, extras


def test_instantiate_nested_kwargs_and_globals():
    cfg = OmegaConf.create({"_component_": "Food", "seed": 0, "ingredient": {"_component_": "Spice", "heat": 5}, "extras": [{"_component_": "Spice", "heat": 1}]})
    food = config.instantiate(cfg, seed=42)
    assert food.seed == 42 and food.ingredient.heat == 5 and food.extras[0].heat == 1
    food = config.instantiate(cfg, ingredient={"_component_": "Spice", "heat": 10})
    assert food.ingredient.heat == 10
    lin = config.instantiate({"_component_": "torch.nn.Linear", "in_features": 2, "out_features": 3})
    assert isinstance(lin, torch.nn.Linear)
    # reference-style dotted paths resolve to this package
    rn = config.instantiate({"_component_": "torchtune.modules.RMSNorm", "dim": 8})
    assert type(rn).__name__ == "RMSNorm"
    with pytest.raises(InstantiationError):
        config.instantiate({"a": 1})
    assert config.instantiate(None) is None


def test_instantiate_positional_and_parent_interpolation():
    root = OmegaConf.create({"dim": 16, "norm": {"_component_": "torchtune_b200.modules.RMSNorm", "dim": "${dim}"}})
    assert config.instantiate(root.norm).scale.numel() == 16
    opt_cfg = OmegaConf.create({"_component_": "torch.optim.SGD", "lr": 0.1})
    p = torch.nn.Parameter(torch.zeros(2))
    opt = config.instantiate(opt_cfg, [p])
    assert opt.param_groups[0]["lr"] == 0.1


def test_validate_reports_all_errors():
    good = OmegaConf.create({"m": {"_component_": "torch.nn.Linear", "in_features": 1, "out_features": 2}, "d": {"_component_": "torch.nn.Linear", "out_features": 2}})
    config.validate(good)  # missing required arg is tolerated
    bad = OmegaConf.create({"m": {"_component_": "torch.nn.Linear", "in_features": 1, "out_features": 2, "bogus": 3}, "n": {"_component_": "torch.nn.ReLU", "zzz": 1}})
    with pytest.raises(ConfigError) as exc:
        config.validate(bad)
    assert len(exc.value.errors) == 2


def test_to_yaml_save_and_resolver(tmp_path):
    cfg = OmegaConf.create({"b": 2, "a": "${b}"})
    text = OmegaConf.to_yaml(cfg, resolve=True, sort_keys=True)
    assert text.index("a:") < text.index("b:") and "a: 2" in text
    OmegaConf.save(cfg, tmp_path / "c.yaml")
    assert OmegaConf.load(tmp_path / "c.yaml").a == 2
    OmegaConf.register_new_resolver("eval", eval, replace=True)
    assert OmegaConf.create({"x": "${eval:'2*3'}"}).x == 6


def test_every_shipped_config_is_well_formed():
    from torchtune_b200._recipe_registry import CONFIGS_DIR

    files = sorted(CONFIGS_DIR.rglob("*.yaml"))
    assert files
    for f in files:
        config.validate(OmegaConf.load(f))
