"""One registry from an architecture's name (config.json ``architectures[0]``, or the single name
under ``architecture``) to its typed configuration and its model description.

lite_llama branches on ``model_type`` in two if/elif chains
(lite_llama/executor/model_executor.py:141-153,170-181); here both the configuration class and
the function that turns it into a ``ModelSpec`` hang on one name.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Dict, Union


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[Dict[str, Any]], Any]
    spec_from_config: Callable[..., Any]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict, spec_from_config) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_from_dict, spec_from_config)


def known_architectures():
    return sorted(_ARCHITECTURES)


def resolve_architecture(config: Dict[str, Any]) -> Architecture:
    archs = config.get("architectures") or config.get("architecture")
    if not archs:
        raise KeyError(f"config.json has neither 'architectures' nor 'architecture'; known: {known_architectures()}")
    name = archs if isinstance(archs, str) else archs[0]
    if name not in _ARCHITECTURES:
        raise KeyError(f"architecture {name!r} is not registered; known: {known_architectures()}")
    return _ARCHITECTURES[name]


def read_config_json(folder: Union[str, Path]) -> Dict[str, Any]:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"{path} not found")
    return json.loads(path.read_text())


def _register_builtin() -> None:
    from .llama import LlamaConfig
    from ..models.llama import llama_spec
    register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, llama_spec)
    from .tibepel import TibepelConfig
    from ..models.tibepel import tibepel_spec
    register_architecture("Tibepel", TibepelConfig.from_dict, tibepel_spec)
    from .lilenex import LilenexConfig
    from ..models.lilenex import lilenex_spec
    register_architecture("Lilenex", LilenexConfig.from_dict, lilenex_spec)
    from .sogalix import SogalixConfig
    from ..models.sogalix import sogalix_spec
    register_architecture("Sogalix", SogalixConfig.from_dict, sogalix_spec)
    from .podizen import PodizenConfig
    from ..models.podizen import podizen_spec
    register_architecture("Podizen", PodizenConfig.from_dict, podizen_spec)


_register_builtin()
