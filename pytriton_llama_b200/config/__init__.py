from .llama import ConfigError, LlamaConfig, RopeScaling  # noqa: F401
from .engine import EngineConfig  # noqa: F401
from .tibepel import TibepelConfig  # noqa: F401
from .lilenex import LilenexConfig  # noqa: F401
from .sogalix import SogalixConfig  # noqa: F401
from .podizen import PodizenConfig  # noqa: F401
from .registry import (known_architectures, read_config_json, register_architecture,  # noqa: F401
                       resolve_architecture)
