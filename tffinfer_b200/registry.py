"""One registry from names to creators, in the manner of the reference's ModuleFactory
(include/ModuleFactory.h:144-226: type string x key -> creator; a lookup of an
unknown key returns nullptr there, here it raises and lists what is registered).

Two kinds of entries exist:

* architectures: ``architectures[0]`` of config.json -> :class:`Architecture`
  (how to read the typed configuration, and how to turn it into a model description
  made of parts) -- cf. ``REGISTER_MODULE_OBJECT(QWen3Creator, ModelCreatorBase,
  MODEL_CREATOR_FLAG, "qwen3")`` at src/core/model/qwen3/QWen3Creator.cpp:11-12;
* parts: (family, kind) -> class, with family one of ``mixer``, ``feed_forward``,
  ``norm``, ``position``, ``block``.

Registration is open: code outside the package (a test, a plug-in) may register a
new part or a whole architecture without touching any file of the framework.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Tuple

PART_FAMILIES = ("mixer", "feed_forward", "norm", "position", "block")


class RegistryError(KeyError):
    def __str__(self) -> str:  # KeyError quotes its message otherwise
        return self.args[0] if self.args else ""


@dataclass(frozen=True)
class Architecture:
    """What a model family has to provide.

    read_config(json_dict) -> ModelConfig       typed configuration from config.json
    describe(config)       -> ModelDescription  the layers as data (parts/description.py)
    """
    name: str
    read_config: Callable[[Dict[str, Any]], Any]
    describe: Callable[[Any], Any]


_ARCHITECTURES: Dict[str, Architecture] = {}
_PARTS: Dict[Tuple[str, str], type] = {}


def register_architecture(name: str, read_config, describe, *, replace: bool = False) -> Architecture:
    if name in _ARCHITECTURES and not replace:
        raise RegistryError(f"architecture '{name}' is already registered")
    arch = Architecture(name, read_config, describe)
    _ARCHITECTURES[name] = arch
    return arch


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        known = ", ".join(sorted(_ARCHITECTURES)) or "(none)"
        raise RegistryError(f"unknown architecture '{name}'; registered: {known}") from None


def registered_architectures():
    return sorted(_ARCHITECTURES)


def register_part(family: str, kind: str, *, replace: bool = False):
    """Class decorator: ``@register_part("mixer", "gqa_attention")``."""
    if family not in PART_FAMILIES:
        raise RegistryError(f"unknown part family '{family}'; families: {', '.join(PART_FAMILIES)}")

    def deco(cls):
        key = (family, kind)
        if key in _PARTS and not replace and _PARTS[key] is not cls:
            raise RegistryError(f"{family} '{kind}' is already registered")
        _PARTS[key] = cls
        cls.family = family
        cls.kind = kind
        return cls
    return deco


def get_part(family: str, kind: str) -> type:
    try:
        return _PARTS[(family, kind)]
    except KeyError:
        known = ", ".join(sorted(k for f, k in _PARTS if f == family)) or "(none)"
        raise RegistryError(f"unknown {family} '{kind}'; registered: {known}") from None


def registered_parts(family: str):
    return sorted(k for f, k in _PARTS if f == family)
