"""Immutable, strictly validated configuration objects.

Same contract as the reference's ``BaseConfig`` (src/scaling/core/config/base.py:39-165): pydantic
v2 models that forbid unknown keys and are frozen after construction, JSON-compatible dict/str/yaml
round trips, a recursive overwrite that extends the ``training_groups`` list element-wise, and a
commented template generator (YAML files are "JSON with comments").
"""

from __future__ import annotations

import json
from enum import Enum
from pathlib import Path
from typing import Any, Optional, Type, TypeVar, Union

import yaml
from pydantic import BaseModel, ConfigDict

T = TypeVar("T", bound="BaseConfig")

# keys whose list values are merged item by item instead of being replaced
_ELEMENTWISE_LIST_KEYS = ("training_groups",)


def overwrite_recursive(target: dict, updates: dict) -> None:
    """Merge ``updates`` into ``target`` in place (nested dicts merged, other values replaced)."""
    for key, new in updates.items():
        if isinstance(new, dict):
            sub = target.get(key)
            if not isinstance(sub, dict):
                sub = {}
                target[key] = sub
            overwrite_recursive(sub, new)
        elif isinstance(new, list) and key in _ELEMENTWISE_LIST_KEYS:
            cur = target.setdefault(key, [])
            while len(cur) < len(new):
                cur.append({})
            for i, item in enumerate(new):
                overwrite_recursive(cur[i], item)
        else:
            target[key] = new


def _plain(value: Any) -> Any:
    if isinstance(value, dict):
        return {k: _plain(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return [_plain(v) for v in value]
    if isinstance(value, Path):
        return str(value)
    if isinstance(value, Enum):
        return value.value
    return value


class BaseConfig(BaseModel):
    model_config = ConfigDict(extra="forbid", frozen=True, protected_namespaces=())

    # ---- conversions
    def as_dict(self) -> dict[str, Any]:
        return _plain(self.model_dump())

    def as_str(self) -> str:
        return json.dumps(self.as_dict())

    @classmethod
    def from_dict(cls: Type[T], d: dict, overwrite_values: Optional[dict] = None) -> T:
        if overwrite_values is not None:
            overwrite_recursive(d, overwrite_values)
        return cls(**d)

    @classmethod
    def from_str(cls: Type[T], s: str) -> T:
        return cls.from_dict(json.loads(s))

    @classmethod
    def from_yaml(cls: Type[T], yml_filename: Union[str, Path], overwrite_values: Optional[dict] = None) -> T:
        with open(yml_filename, encoding="utf-8") as f:
            d = yaml.safe_load(f) or {}
        return cls.from_dict(d, overwrite_values)

    def save(self, out_file: Union[str, Path], indent: int = 4) -> None:
        with open(out_file, "w", encoding="utf-8") as f:
            json.dump(self.as_dict(), f, indent=indent)

    # ---- template
    @classmethod
    def get_template_str(cls, indent: int = 4, level: int = 1) -> str:
        pad = " " * indent * level

        def comment(text: Optional[str]) -> str:
            if not text or not text.strip():
                return ""
            return "".join(f"{pad}# {line}\n" for line in text.strip().split("\n"))

        lines = ["{\n", comment(cls.__name__), comment(cls.__doc__)]
        names = list(cls.model_fields.keys())
        for i, name in enumerate(names):
            info = cls.model_fields[name]
            lines.append(pad + "\n")
            lines.append(comment(info.description))
            entry = f'{pad}"{name}": '
            default = info.default
            if isinstance(default, BaseConfig):
                entry += type(default).get_template_str(indent=indent, level=level + 1)
            elif isinstance(default, Enum):
                entry += json.dumps(default.value)
            elif default is not None and repr(default) != "PydanticUndefined":
                try:
                    entry += json.dumps(_plain(default))
                except TypeError:
                    entry += "null"
            if i != len(names) - 1:
                entry += ","
            lines.append(entry + "\n")
        lines.append(" " * indent * (level - 1) + "}")
        return "".join(lines)

    @classmethod
    def save_template(cls, out_file: Union[str, Path], indent: int = 4) -> None:
        with open(out_file, "w", encoding="utf-8") as f:
            f.write(cls.get_template_str(indent=indent))
