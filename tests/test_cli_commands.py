"""`tune ls / cp / cat / validate / run` driven in-process through the real parser."""
import sys

import pytest
import yaml

from torchtune_b200._cli import tune
from torchtune_b200._recipe_registry import get_all_recipes


def _tune(monkeypatch, argv):
    monkeypatch.setattr(sys, "argv", ["tune"] + argv)
    parser = tune.TuneCLIParser()
    parser.run(parser.parse_args())


def test_no_subcommand_prints_help(monkeypatch, capsys):
    _tune(monkeypatch, [])
    out = capsys.readouterr().out
    assert "subcommands" in out and "download" in out and "validate" in out


def test_ls_lists_every_recipe_and_config(monkeypatch, capsys):
    _tune(monkeypatch, ["ls"])
    out = capsys.readouterr().out
    lines = out.splitlines()
    assert lines[0].split() == ["RECIPE", "CONFIG"]
    for recipe in get_all_recipes():
        assert recipe.name in out
        for cfg in recipe.configs:
            assert cfg.name in out
    # a recipe's name is printed once, on the row of its first config
    assert sum(1 for line in lines if line.startswith("full_finetune_single_device ")) == 1


def test_cp_config_and_recipe(monkeypatch, capsys, tmp_path):
    dest = tmp_path / "mine.yaml"
    _tune(monkeypatch, ["cp", "llama3_1/8B_full", str(dest)])
    assert "Copied file to" in capsys.readouterr().out
    assert yaml.safe_load(dest.read_text())["model"]["_component_"].endswith("llama3_1_8b")

    # the right suffix is put on when the destination has another
    _tune(monkeypatch, ["cp", "full_finetune_single_device", str(tmp_path / "recipe.txt")])
    assert "tune-recipe:" in (tmp_path / "recipe.py").read_text()
    capsys.readouterr()

    # --no-clobber leaves an existing file alone
    dest.write_text("keep: me\n")
    _tune(monkeypatch, ["cp", "llama3_1/8B_full", str(dest), "--no-clobber"])
    assert "not overwriting" in capsys.readouterr().out and dest.read_text() == "keep: me\n"

    # a missing parent is an error unless --make-parents is given
    deep = tmp_path / "a" / "b" / "c.yaml"
    with pytest.raises(SystemExit):
        _tune(monkeypatch, ["cp", "llama3_1/8B_full", str(deep)])
    assert "--make-parents" in capsys.readouterr().err
    _tune(monkeypatch, ["cp", "llama3_1/8B_full", str(deep), "--make-parents"])
    assert deep.exists()

    with pytest.raises(SystemExit):
        _tune(monkeypatch, ["cp", "no_such_thing", str(tmp_path / "x.yaml")])
    assert "Invalid file name" in capsys.readouterr().err


def test_cat_prints_yaml_sorted_on_request(monkeypatch, capsys, tmp_path):
    _tune(monkeypatch, ["cat", "llama3_1/8B_full"])
    plain = capsys.readouterr().out
    data = yaml.safe_load(plain)
    assert data["model"]["_component_"].endswith("llama3_1_8b")
    _tune(monkeypatch, ["cat", "llama3_1/8B_full", "--sort"])
    keys = [line.split(":")[0] for line in capsys.readouterr().out.splitlines() if line and not line.startswith((" ", "-"))]
    assert keys == sorted(keys) and list(data) != sorted(data)

    local = tmp_path / "local.yaml"
    local.write_text("b: 1\na: 2\n")
    _tune(monkeypatch, ["cat", str(local)])
    assert capsys.readouterr().out.splitlines()[:2] == ["b: 1", "a: 2"]

    with pytest.raises(SystemExit):
        _tune(monkeypatch, ["cat", "full_finetune_single_device"])
    assert "is a recipe, not a config" in capsys.readouterr().err
    with pytest.raises(SystemExit):
        _tune(monkeypatch, ["cat", "nowhere/none"])
    assert "not found or invalid" in capsys.readouterr().err


def test_validate_accepts_good_and_names_the_bad_argument(monkeypatch, capsys, tmp_path):
    good = tmp_path / "good.yaml"
    good.write_text("layer:\n  _component_: torch.nn.Linear\n  in_features: 4\n  out_features: 2\n")
    _tune(monkeypatch, ["validate", str(good)])
    assert "well-formed" in capsys.readouterr().out
    _tune(monkeypatch, ["validate", "llama3_1/8B_full"])  # a built-in name works as well as a path
    assert "well-formed" in capsys.readouterr().out

    bad = tmp_path / "bad.yaml"
    bad.write_text("layer:\n  _component_: torch.nn.Linear\n  in_features: 4\n  out_features: 2\n  not_an_argument: 1\n")
    with pytest.raises(SystemExit):
        _tune(monkeypatch, ["validate", str(bad)])
    assert "not_an_argument" in capsys.readouterr().err


def test_run_needs_a_config_and_refuses_torchrun_for_single_device_recipes(monkeypatch, capsys):
    with pytest.raises(SystemExit):
        _tune(monkeypatch, ["run", "full_finetune_single_device"])
    assert "'--config' argument is required" in capsys.readouterr().err
    with pytest.raises(SystemExit):
        _tune(monkeypatch, ["run", "--nproc_per_node", "2", "full_finetune_single_device", "--config", "llama3_1/8B_full_single_device"])
    assert "does not support distributed training" in capsys.readouterr().err


def test_run_resolves_builtin_names_and_passes_overrides(monkeypatch, tmp_path):
    seen = {}

    def fake_run_path(script, run_name):
        seen["script"], seen["argv"], seen["run_name"] = script, list(sys.argv), run_name

    monkeypatch.setattr(tune.runpy, "run_path", fake_run_path)
    _tune(monkeypatch, ["run", "full_finetune_single_device", "--config", "llama3_1/8B_full_single_device", "batch_size=3"])
    assert seen["script"].endswith("recipes/full_finetune_single_device.py") and seen["run_name"] == "__main__"
    assert seen["argv"][0] == seen["script"] and seen["argv"][1] == "--config"
    assert seen["argv"][2].endswith("configs/llama3_1/8B_full_single_device.yaml") and seen["argv"][3] == "batch_size=3"

    # a config that is a local path is handed through untouched
    local = tmp_path / "mine.yaml"
    local.write_text("a: 1\n")
    _tune(monkeypatch, ["run", "full_finetune_single_device", "--config", str(local)])
    assert seen["argv"][2] == str(local)

    # a recipe that is not built in is run as a module of the working directory
    mods = {}
    monkeypatch.setattr(tune.runpy, "run_module", lambda name, run_name: mods.update(name=name))
    _tune(monkeypatch, ["run", "my_pkg/my_recipe.py", "--config", str(local)])
    assert mods["name"] == "my_pkg.my_recipe"
