"""One registry from an architecture's name to its configuration class and
model builder.

`config.json` names the architecture in `architectures[0]`; everything in the
framework (loader, engine, trace replay, command line) goes through
`resolve()` to find out what to build.  An unknown name is an error that
lists the known ones, as the reference's registry does
(crates/runtime/src/registry.rs:18-77).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from .base import ConfigError, ConfigReader, read_config_json


class UnknownArchitecture(ConfigError):
    def __init__(self, name: str, known: list[str]):
        super().__init__(f"architecture '{name}' is not registered; known: {', '.join(sorted(known)) or '(none)'}")
        self.name, self.known = name, known


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                      # has from_dict(raw) and to_dict()
    build_spec: Callable[[Any], Any]       # config -> parts.spec.ModelSpec


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class, build_spec, *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def resolve(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise UnknownArchitecture(name, list(_ARCHITECTURES)) from None


def load_config(folder_or_file):
    """(architecture entry, typed config) for a model folder."""
    raw = read_config_json(folder_or_file)
    arch = resolve(ConfigReader(raw).architecture())
    return arch, arch.config_class.from_dict(raw)
