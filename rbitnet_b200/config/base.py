"""Typed configuration: the base class every architecture's configuration derives from.

A configuration is read from the architecture's own ``config.json`` keys.  No
size, and no constant that ``config.json`` gives, stands anywhere else in the
package: parts receive their sizes as parameters from the architecture's
builder, which reads them here.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, fields, asdict
from pathlib import Path
from typing import Any, ClassVar, Mapping


class ConfigError(ValueError):
    """A config.json that is missing a key, or whose values do not fit together."""


@dataclass
class ModelConfig:
    """Base of all architecture configurations.

    Subclasses declare their fields as dataclass fields named after the
    config.json keys they are read from, set ``architecture`` to the name in
    config.json's ``architectures`` list, and implement ``validate``.
    """

    architecture: ClassVar[str] = ""
    #: config.json keys that must be present (the rest have defaults)
    required: ClassVar[tuple] = ()
    #: config.json keys that may be present only with the given value, because
    #: the architecture has no such path
    pinned: ClassVar[Mapping[str, Any]] = {}

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]):
        missing = [k for k in cls.required if d.get(k) is None]
        if missing:
            raise ConfigError(f"config.json: missing {', '.join(missing)}")
        for key, allowed in cls.pinned.items():
            if key in d and d[key] is not None and d[key] != allowed:
                raise ConfigError(
                    f"config.json: {key}={d[key]!r} is not supported by {cls.architecture} "
                    f"(only {allowed!r})")
        known = {f.name for f in fields(cls)}
        kwargs = {k: d[k] for k in known if k in d and d[k] is not None}
        cfg = cls(**kwargs)
        cfg.validate()
        return cfg

    def validate(self) -> None:  # pragma: no cover - overridden
        pass

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [self.architecture]
        return d

    def save(self, folder) -> None:
        Path(folder).mkdir(parents=True, exist_ok=True)
        (Path(folder) / "config.json").write_text(json.dumps(self.to_dict(), indent=1))


def read_config_json(folder) -> dict:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no config.json in the model folder")
    try:
        d = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d
