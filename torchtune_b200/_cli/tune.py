"""``tune`` command line: ``run``, ``ls``, ``cp``, ``cat``, ``validate``, ``download``.

Parity: torchtune/_cli/tune.py:18-52, run.py:26-214, ls.py:45-64, cp.py:73-116,
cat.py:92-128, validate.py:50-59, download.py:29-287.
"""
from __future__ import annotations

import argparse
import json
import os
import runpy
import shutil
import sys
import textwrap
from pathlib import Path
from typing import List, Optional, Tuple

import yaml

from torchtune_b200 import config as _config
from torchtune_b200._recipe_registry import CONFIGS_DIR, RECIPES_DIR, Config, Recipe, get_all_recipes


# ---------------------------------------------------------------------------- lookup
def _find_recipe(name: str) -> Optional[Recipe]:
    return next((r for r in get_all_recipes() if r.name == name), None)


def _find_config(name: str, within: Optional[Recipe] = None) -> Optional[Config]:
    pools = ([within] if within is not None else []) + get_all_recipes()
    for r in pools:
        for c in r.configs:
            if c.name == name:
                return c
    return None


# ---------------------------------------------------------------------------- run
def _add_run(sub) -> argparse.ArgumentParser:
    from torch.distributed.run import get_args_parser

    p = sub.add_parser(
        "run",
        prog="tune run",
        help="Run a recipe. For distributed recipes, this supports all torchrun arguments.",
        description="Run a recipe. For distributed recipes, this supports all torchrun arguments.",
        usage="tune run [TORCHRUN-OPTIONS] <recipe> --config <config> [RECIPE-OPTIONS]",
        epilog=textwrap.dedent(
            """\
            examples:
                $ tune run lora_finetune_single_device --config llama3_1/8B_lora_single_device
                $ tune run --nproc_per_node 8 full_finetune_distributed --config llama3_1/8B_full batch_size=4
            """
        ),
        formatter_class=argparse.RawTextHelpFormatter,
    )
    # Re-export every torchrun option; its positional script slots become the recipe.
    for action in get_args_parser()._actions:
        if action.dest == "help":
            continue
        if action.dest == "training_script":
            action.dest = "recipe"
            action.help = "Name or path to recipe to be launched followed by args.\nFor a list of all possible recipes, run `tune ls`."
        elif action.dest == "training_script_args":
            action.dest = "recipe_args"
            action.help = "Args to be passed to the recipe."
        p._add_action(action)
    p.set_defaults(func=lambda a: _run(p, a))
    return p


def _run(parser: argparse.ArgumentParser, args: argparse.Namespace) -> None:
    try:
        cfg_pos = args.recipe_args.index("--config") + 1
        cfg_name = args.recipe_args[cfg_pos]
    except (ValueError, IndexError):
        parser.error("The '--config' argument is required.")
    recipe = _find_recipe(args.recipe)
    builtin = recipe is not None
    if builtin:
        script = str(RECIPES_DIR / recipe.file_path)
    else:
        script = os.path.splitext(args.recipe)[0].replace("/", ".")  # custom recipe → module path
    cfg = _find_config(cfg_name, recipe)
    args.recipe_args[cfg_pos] = str(CONFIGS_DIR / cfg.file_path) if cfg is not None else cfg_name
    args.recipe = script
    sys.path.append(os.getcwd())

    # torchrun options were given iff argv holds more than "<recipe> <recipe args…>"
    launched_distributed = (len(sys.argv) - 2) > (len(args.recipe_args) + 1)
    if launched_distributed:
        if builtin and not recipe.supports_distributed:
            parser.error(f"Recipe {recipe.name} does not support distributed training.Please run without torchrun commands.")
        _run_distributed(args, builtin)
    else:
        sys.argv = [script] + list(args.recipe_args)
        if builtin:
            runpy.run_path(script, run_name="__main__")
        else:
            runpy.run_module(script, run_name="__main__")


def _run_distributed(args: argparse.Namespace, builtin: bool) -> None:
    from torch.distributed.elastic.multiprocessing.errors import record
    from torch.distributed.run import run

    @record
    def launch() -> None:
        print("Running with torchrun...")
        args.training_script = args.recipe
        args.training_script_args = args.recipe_args
        if not args.rdzv_endpoint:
            args.standalone = True
        args.module = not builtin
        run(args)

    launch()


# ---------------------------------------------------------------------------- ls
def _add_ls(sub) -> None:
    p = sub.add_parser("ls", prog="tune ls", help="List all built-in recipes and configs", description="List all built-in recipes and configs")
    p.set_defaults(func=_ls)


def _ls(args: argparse.Namespace) -> None:
    header = f"{'RECIPE':<40} {'CONFIG':<40}"
    print(header)
    for r in get_all_recipes():
        if not r.configs:
            print(f"{r.name:<40} {'<>':<40}")
        for i, c in enumerate(r.configs):
            print(f"{(r.name if i == 0 else ''):<40} {c.name:<40}")


# ---------------------------------------------------------------------------- cp
def _add_cp(sub) -> None:
    p = sub.add_parser("cp", prog="tune cp", usage="tune cp <recipe|config> destination [OPTIONS]", help="Copy a built-in recipe or config to a local path.", description="Copy a built-in recipe or config to a local path.")
    p.add_argument("file", type=str, help="Recipe/config to copy. For a list of all possible options, run `tune ls`")
    p.add_argument("destination", type=Path, help="Location to copy the file to")
    p.add_argument("-n", "--no-clobber", action="store_true", default=False, help="Do not overwrite destination if it already exists")
    p.add_argument("--make-parents", action="store_true", default=False, help="Create parent directories for destination if they do not exist.")
    p.set_defaults(func=lambda a: _cp(p, a))


def _cp(parser: argparse.ArgumentParser, args: argparse.Namespace) -> None:
    dest: Path = args.destination
    src, suffix = None, None
    recipe = _find_recipe(args.file)
    if recipe is not None:
        src, suffix = RECIPES_DIR / recipe.file_path, ".py"
    else:
        cfg = _find_config(args.file)
        if cfg is not None:
            src, suffix = CONFIGS_DIR / cfg.file_path, ".yaml"
    if src is None:
        parser.error(f"Invalid file name: {args.file}. Try `tune ls` to see all available files to copy.")
    if dest.suffix != suffix:
        dest = dest.with_suffix(suffix)
    if args.no_clobber and dest.exists():
        print(f"File already exists at {dest.absolute()}, not overwriting.")
        return
    if args.make_parents:
        dest.parent.mkdir(parents=True, exist_ok=True)
    try:
        shutil.copy2(src, dest)
    except FileNotFoundError:
        parser.error(f"Cannot create regular file: '{dest}'. No such file or directory. If the specified destination's parent directory does not exist and you would like to create it on-the-fly, use the --make-parents flag.")
    print(f"Copied file to {dest.absolute()}")


# ---------------------------------------------------------------------------- cat
def _add_cat(sub) -> None:
    p = sub.add_parser("cat", prog="tune cat", usage="tune cat <config-name> [--sort]", help="Pretty print a config, making it easy to know which parameters you can override with `tune run`.", description="Pretty print a config.")
    p.add_argument("config_name", type=str, help="Name of the config to print")
    p.add_argument("--sort", action="store_true", help="Print the config in sorted order")
    p.set_defaults(func=lambda a: _cat(p, a))


def _cat(parser: argparse.ArgumentParser, args: argparse.Namespace) -> None:
    name = args.config_name
    if _find_recipe(name) is not None:
        parser.error(f"'{name}' is a recipe, not a config. Please use a config name.")
    cfg = _find_config(name)
    if cfg is not None:
        path = CONFIGS_DIR / cfg.file_path
    elif name.endswith(".yaml") and Path(name).exists():
        path = Path(name)
    else:
        parser.error(f"Config '{name}' not found or invalid. Please run 'tune ls' to see the available configs.")
    if not path.exists():
        parser.error(f"Config '{path}' not found.")
    data = yaml.safe_load(path.read_text())
    print(yaml.dump(data, default_flow_style=False, sort_keys=args.sort))


# ---------------------------------------------------------------------------- validate
def _add_validate(sub) -> None:
    p = sub.add_parser("validate", prog="tune validate", usage="tune validate <config>", help="Validate a config and ensure that it is well-formed.", description="Validate a config and ensure that it is well-formed.")
    p.add_argument("config", type=Path, help="Path to a config to validate.")
    p.set_defaults(func=lambda a: _validate(p, a))


def _validate(parser: argparse.ArgumentParser, args: argparse.Namespace) -> None:
    path = args.config
    if not Path(path).exists():
        known = _find_config(str(path))
        if known is not None:
            path = CONFIGS_DIR / known.file_path
    cfg = _config.OmegaConf.load(path)
    try:
        _config.validate(cfg)
    except _config.ConfigError as exc:
        parser.error(str(exc))
    print("Config is well-formed!")


# ---------------------------------------------------------------------------- download
def _add_download(sub) -> None:
    p = sub.add_parser("download", prog="tune download", usage="tune download <repo-id> [OPTIONS]", help="Download a model from the Hugging Face Hub or Kaggle Model Hub.", description="Download a model from the Hugging Face Hub or Kaggle Model Hub.")
    p.add_argument("repo_id", type=str, help="Name of the repository on Hugging Face Hub or model handle on Kaggle Model Hub.")
    p.add_argument("--output-dir", type=Path, required=False, default=None, help="Directory in which to save the model. Defaults to `/tmp/<model_name>`.")
    p.add_argument("--hf-token", type=str, required=False, default=os.getenv("HF_TOKEN", None), help="Hugging Face API token. Needed for gated models like Llama2.")
    p.add_argument("--ignore-patterns", type=str, required=False, help="If provided, files matching any of the patterns are not downloaded. Example: '*.safetensors'.")
    p.add_argument("--source", type=str, required=False, default="huggingface", choices=["huggingface", "kaggle"], help="If provided, downloads model weights from the provided repo_id on the designated source hub.")
    p.add_argument("--kaggle-username", type=str, required=False, help="Kaggle username for authentication.")
    p.add_argument("--kaggle-api-key", type=str, required=False, help="Kaggle API key.")
    p.set_defaults(func=lambda a: _download(p, a))


def _download(parser: argparse.ArgumentParser, args: argparse.Namespace) -> None:
    out = args.output_dir
    if out is None:
        out = Path("/tmp") / args.repo_id.split("/")[-1]
    if args.source == "kaggle":
        try:
            import kagglehub
        except ImportError:
            parser.error("kagglehub is required for --source kaggle; install it with `pip install kagglehub`.")
        if args.kaggle_username or args.kaggle_api_key:
            os.environ.setdefault("KAGGLE_USERNAME", args.kaggle_username or "")
            os.environ.setdefault("KAGGLE_KEY", args.kaggle_api_key or "")
        try:
            path = kagglehub.model_download(args.repo_id)
        except Exception as exc:
            parser.error(f"Failed to download '{args.repo_id}' from Kaggle: {exc}")
        print("Successfully downloaded model repo and wrote to the following locations:", path, sep="\n")
        return
    try:
        from huggingface_hub import snapshot_download
        from huggingface_hub.utils import GatedRepoError, RepositoryNotFoundError
    except ImportError:
        parser.error("huggingface_hub is required for downloads")
    print(f"Ignoring files matching the following patterns: {args.ignore_patterns}")
    try:
        true_dir = snapshot_download(args.repo_id, local_dir=str(out), ignore_patterns=args.ignore_patterns, token=args.hf_token)
    except GatedRepoError:
        parser.error("It looks like you are trying to access a gated repository. Please ensure you have access to the repository" + (" and have provided the proper Hugging Face API token using the option `--hf-token` or by running `huggingface-cli login`." if not args.hf_token else "."))
    except RepositoryNotFoundError:
        parser.error(f"Repository '{args.repo_id}' not found on the Hugging Face Hub.")
    except Exception as exc:
        msg = f"Failed to download {args.repo_id} with error: '{exc}' and traceback: {exc.__traceback__}"
        parser.error(msg)
    # remembered so that PEFT adapter configs can name their base model
    (Path(true_dir) / "original_repo_id.json").write_text(json.dumps({"repo_id": args.repo_id}))
    print("Successfully downloaded model repo and wrote to the following locations:", *sorted(str(p) for p in Path(true_dir).iterdir()), sep="\n")


# ---------------------------------------------------------------------------- entry
class TuneCLIParser:
    """Top-level parser; with no sub-command it prints the help text."""

    def __init__(self) -> None:
        self._parser = argparse.ArgumentParser(prog="tune", description="Welcome to the torchtune CLI!", add_help=True)
        self._parser.set_defaults(func=lambda args: self._parser.print_help())
        sub = self._parser.add_subparsers(title="subcommands")
        _add_download(sub)
        _add_ls(sub)
        _add_cp(sub)
        _add_run(sub)
        _add_validate(sub)
        _add_cat(sub)

    def parse_args(self) -> argparse.Namespace:
        return self._parser.parse_args()

    def run(self, args: argparse.Namespace) -> None:
        args.func(args)


def main() -> None:
    parser = TuneCLIParser()
    parser.run(parser.parse_args())


if __name__ == "__main__":
    main()
