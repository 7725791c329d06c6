from ._errors import ConfigError, InstantiationError
from ._instantiate import instantiate
from ._node import DictConfig, ListConfig, OmegaConf
from ._parse import parse
from ._utils import log_config
from ._validate import validate

__all__ = [
    "instantiate",
    "parse",
    "log_config",
    "validate",
    "DictConfig",
    "ListConfig",
    "OmegaConf",
    "ConfigError",
    "InstantiationError",
]
