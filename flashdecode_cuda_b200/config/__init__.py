"""Configurations: reading ``config.json`` and the named presets.

``load_config`` picks the configuration class through the architecture
registry, from ``config.json["architectures"][0]``.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Dict, List, Union

from ..registry import architecture
from .qwen2 import ConfigError, Qwen2Config

PRESET_DIR = Path(__file__).resolve().parent / "presets"


def preset_names() -> List[str]:
    return sorted(p.stem for p in PRESET_DIR.glob("*.json"))


def preset_dict(name: str) -> Dict[str, Any]:
    """The ``config.json`` dictionary of a named preset (data files under
    ``config/presets/``; sizes live there, not in code)."""
    path = PRESET_DIR / f"{name}.json"
    if not path.exists():
        raise ConfigError(f"unknown preset {name!r}; presets: {preset_names()}")
    return json.loads(path.read_text())


def config_from_dict(cfg: Dict[str, Any]):
    archs = cfg.get("architectures")
    if not archs:
        raise ConfigError("config.json has no 'architectures' entry to choose the model by")
    try:
        arch = architecture(archs[0])
    except KeyError as e:
        raise ConfigError(str(e.args[0])) from None
    return arch.config_cls.from_dict(cfg)


def load_config(source: Union[str, Path, Dict[str, Any]]):
    """A typed configuration from a model folder, a ``config.json`` path, a
    preset name or a dictionary."""
    if isinstance(source, dict):
        return config_from_dict(source)
    p = Path(source)
    if p.is_dir():
        p = p / "config.json"
    if p.exists():
        try:
            return config_from_dict(json.loads(p.read_text()))
        except json.JSONDecodeError as e:
            raise ConfigError(f"{p}: not valid JSON: {e}") from None
    if isinstance(source, str) and (PRESET_DIR / f"{source}.json").exists():
        return config_from_dict(preset_dict(source))
    raise ConfigError(f"no config.json at {source!r} and no preset of that name; presets: {preset_names()}")


__all__ = ["ConfigError", "Qwen2Config", "load_config", "config_from_dict", "preset_dict", "preset_names"]
