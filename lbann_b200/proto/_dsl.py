"""Tiny constructors used by the schema tables (see ``schema.py``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class EnumDef:
    name: str
    values: list  # [(name, number)]


@dataclass
class FieldDef:
    name: str
    number: int
    type: str
    repeated: bool = False
    optional: bool = False
    oneof: Optional[str] = None


@dataclass
class MessageDef:
    name: str
    fields: List[FieldDef]
    enums: List[EnumDef] = field(default_factory=list)
    nested: List["MessageDef"] = field(default_factory=list)


@dataclass
class FileDef:
    name: str
    imports: List[str]
    messages: List[MessageDef]
    enums: List[EnumDef] = field(default_factory=list)


def E(name: str, values: str) -> EnumDef:
    out = []
    for item in values.split():
        k, v = item.split("=")
        out.append((k, int(v)))
    return EnumDef(name, out)


def _field(spec: str) -> FieldDef:
    parts = spec.split()
    name, num = parts[0].split("=")
    f = FieldDef(name, int(num), parts[1])
    for extra in parts[2:]:
        if extra == "*":
            f.repeated = True
        elif extra == "?":
            f.optional = True
        elif extra.startswith("|"):
            f.oneof = extra[1:]
    return f


def M(name: str, fields, enums=None, nested=None) -> MessageDef:
    return MessageDef(name, [_field(f) for f in fields], list(enums or []), list(nested or []))


def F(name: str, imports, messages, enums=None) -> FileDef:
    return FileDef(name, list(imports), list(messages), list(enums or []))
