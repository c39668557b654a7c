"""One registry from an architecture's name to its model.

A config.json names its architecture under ``architectures[0]`` (a class name such as
``Qwen3ForCausalLM``), ``model_type`` (``qwen3``) or ``architecture`` (``Datasun``, ``Bepilorn``, ``Munerax``, ``Kikelorn``).  Any of them selects the entry; the lookup is
exact and case-sensitive, and an unknown name is answered with the list of known ones, as in
the reference (crates/bfi-models/src/arch.rs:70-91).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Tuple

from .config.base import ConfigError
from .parts.base import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any
    describe: Callable[[Dict[str, Any]], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(names: Tuple[str, ...], arch: Architecture) -> None:
    for n in names:
        if n in _ARCHITECTURES and _ARCHITECTURES[n] is not arch:
            raise ValueError(f"architecture name '{n}' is already registered")
        _ARCHITECTURES[n] = arch


def unregister_architecture(*names: str) -> None:
    for n in names:
        _ARCHITECTURES.pop(n, None)


def registered_architectures() -> List[str]:
    return sorted(_ARCHITECTURES)


def architecture_for(config: Dict[str, Any]) -> Architecture:
    candidates: List[str] = []
    archs = config.get("architectures")
    if isinstance(archs, (list, tuple)):
        candidates += [a for a in archs if isinstance(a, str)]
    for key in ("model_type", "architecture"):
        if isinstance(config.get(key), str):
            candidates.append(config[key])
    if not candidates:
        raise ConfigError("config.json names no architecture (keys 'architectures', 'model_type', 'architecture'); "
                          f"registered: {registered_architectures()}")
    for c in candidates:
        if c in _ARCHITECTURES:
            return _ARCHITECTURES[c]
    raise ConfigError(f"unsupported architecture '{candidates[0]}'; registered: {registered_architectures()}")


def describe_model(config: Dict[str, Any]) -> ModelSpec:
    return architecture_for(config).describe(config)


def _register_builtin() -> None:
    from .architectures import qwen3
    from .config.qwen3 import Qwen3Config
    register_architecture(("qwen3", "Qwen3ForCausalLM"),
                          Architecture(name="qwen3", config_class=Qwen3Config, describe=qwen3.describe))
    from .architectures import datasun
    from .config.datasun import DatasunConfig
    register_architecture(("Datasun", "datasun"),
                          Architecture(name="datasun", config_class=DatasunConfig, describe=datasun.describe))
    from .architectures import bepilorn
    from .config.bepilorn import BepilornConfig
    register_architecture(("Bepilorn", "bepilorn"),
                          Architecture(name="bepilorn", config_class=BepilornConfig, describe=bepilorn.describe))
    from .architectures import munerax
    from .config.munerax import MuneraxConfig
    register_architecture(("Munerax", "munerax"),
                          Architecture(name="munerax", config_class=MuneraxConfig, describe=munerax.describe))
    from .architectures import kikelorn
    from .config.kikelorn import KikelornConfig
    register_architecture(("Kikelorn", "kikelorn"),
                          Architecture(name="kikelorn", config_class=KikelornConfig, describe=kikelorn.describe))


_register_builtin()
