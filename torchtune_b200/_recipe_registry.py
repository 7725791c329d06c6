"""Recipe / config registry built by scanning the packaged ``recipes`` tree.

The reference keeps a ~700-line literal list (torchtune/_recipe_registry.py:24-700).  Here
every recipe script declares itself with a header comment ``# tune-recipe:
distributed=<true|false>`` and every YAML names the recipes it belongs to with
``# tune-config: <recipe>[, <recipe>…]``; the registry is the result of reading those
headers.  A config's name is its path below ``recipes/configs`` without ``.yaml``.
"""
from __future__ import annotations

import functools
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List

ROOT = Path(__file__).resolve().parent.parent
RECIPES_DIR = ROOT / "recipes"
CONFIGS_DIR = RECIPES_DIR / "configs"


@dataclass
class Config:
    name: str
    file_path: str


@dataclass
class Recipe:
    name: str
    file_path: str
    configs: List[Config] = field(default_factory=list)
    supports_distributed: bool = False


_RECIPE_HDR = re.compile(r"^#\s*tune-recipe:\s*distributed=(true|false)", re.I | re.M)
_CONFIG_HDR = re.compile(r"^#\s*tune-config:\s*(.+)$", re.I | re.M)


def _head(path: Path, n: int = 2048) -> str:
    with open(path, "r", errors="ignore") as f:
        return f.read(n)


@functools.lru_cache(maxsize=1)
def _scan() -> Dict[str, Recipe]:
    recipes: Dict[str, Recipe] = {}
    if not RECIPES_DIR.is_dir():
        return recipes
    for py in sorted(RECIPES_DIR.rglob("*.py")):
        m = _RECIPE_HDR.search(_head(py))
        if not m:
            continue
        rel = py.relative_to(RECIPES_DIR)
        name = str(rel.with_suffix(""))
        recipes[name] = Recipe(name=name, file_path=str(rel), supports_distributed=m.group(1).lower() == "true")
    if CONFIGS_DIR.is_dir():
        for y in sorted(CONFIGS_DIR.rglob("*.yaml")):
            m = _CONFIG_HDR.search(_head(y))
            if not m:
                continue
            rel = y.relative_to(CONFIGS_DIR)
            cfg = Config(name=str(rel.with_suffix("")), file_path=str(rel))
            for owner in (s.strip() for s in m.group(1).split(",")):
                if owner in recipes:
                    recipes[owner].configs.append(cfg)
    return recipes


def get_all_recipes() -> List[Recipe]:
    return list(_scan().values())
