"""The two registries of the library.

* ``ARCHITECTURES``: the name in ``config.json["architectures"][0]`` -> how to
  read that architecture's configuration and how to describe its model as a
  blueprint of parts.  davidjoyme/flashdecode-cuda has one engine class for
  its one architecture (engine/model.py:74); here the model class is always
  chosen through this table.
* ``PARTS``: (kind, name) -> the class that implements a part.  Kinds are
  ``embedding``, ``position``, ``norm``, ``mixer``, ``feed_forward``, ``block``
  and ``head``.  A blueprint names parts by (kind, name); nothing else in the
  engine knows a part's class.

A new architecture or part is added by calling ``register_architecture`` /
``register_part`` (usually as a decorator) from any module that is imported
before the model is built; no file of the framework changes.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Tuple, Type

PART_KINDS = ("embedding", "position", "norm", "mixer", "feed_forward", "block", "head")


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type            # has classmethod from_dict(dict) and method to_dict()
    blueprint: Callable         # config -> engine.blueprint.ModelBlueprint


ARCHITECTURES: Dict[str, Architecture] = {}
PARTS: Dict[Tuple[str, str], type] = {}


def register_architecture(name: str, config_cls: type, blueprint: Callable) -> None:
    if name in ARCHITECTURES:
        raise ValueError(f"architecture {name!r} is already registered")
    ARCHITECTURES[name] = Architecture(name, config_cls, blueprint)


def architecture(name: str) -> Architecture:
    try:
        return ARCHITECTURES[name]
    except KeyError:
        raise KeyError(f"unknown architecture {name!r}; registered: {sorted(ARCHITECTURES)}") from None


def register_part(kind: str, name: str) -> Callable[[Type], Type]:
    if kind not in PART_KINDS:
        raise ValueError(f"unknown part kind {kind!r}; kinds: {PART_KINDS}")

    def deco(cls):
        if (kind, name) in PARTS:
            raise ValueError(f"part {kind}/{name} is already registered")
        PARTS[(kind, name)] = cls
        return cls
    return deco


def part_class(kind: str, name: str) -> type:
    try:
        return PARTS[(kind, name)]
    except KeyError:
        have = sorted(n for k, n in PARTS if k == kind)
        raise KeyError(f"no {kind} part named {name!r}; registered: {have}") from None
