"""Config base class and command line.

Behaviour kept from the reference's config system (docs/configuration.md:24-144,
packages/prime-rl-configs/src/prime_rl/utils/config.py:6-22):

* precedence: field defaults < ``@ file.toml`` (several files deep-merge left to right) <
  dotted kebab-case flags (``--model.seq-len 4096``);
* booleans: ``--flag`` / ``--no-flag`` (also ``--flag true|false``);
* the string ``"None"`` means null;
* a bare flag naming an optional sub-config (``--model.lora``) materialises it with defaults,
  ``--no-model.lora`` (or ``--model.lora None``) removes it;
* discriminated unions select on ``type``;
* ``--dry-run`` is handled by the entrypoints after the resolved config was dumped.
"""

from __future__ import annotations

import json
import sys
import tomllib
import types
import typing
from pathlib import Path
from typing import Any, TypeVar, Union, get_args, get_origin

from pydantic import BaseModel, ConfigDict, model_validator

T = TypeVar("T", bound="BaseConfig")


class BaseConfig(BaseModel):
    model_config = ConfigDict(extra="forbid", validate_assignment=False, validate_default=False,
                              arbitrary_types_allowed=True, populate_by_name=True)

    @model_validator(mode="before")
    @classmethod
    def _default_union_tags(cls, data):
        # {"optim": {"lr": 1e-5}} keeps the default optimizer's ``type``; the string "None" (how TOML files
        # and flags spell null, TOML having no null) clears any field that may be None
        if isinstance(data, dict):
            data = inject_union_defaults(cls, dict(data), recurse=False)
            for k, v in list(data.items()):
                if v == "None" and isinstance(v, str):
                    fld = cls.model_fields.get(k)
                    if fld is not None and type(None) in _flatten_union(fld.annotation):
                        data[k] = None
        return data

    def to_json(self, **kw) -> str:
        """JSON dump that keeps nulls, so that a resolved config re-parses to itself."""
        return self.model_dump_json(indent=2, **kw)

    def dump(self, path: Path) -> None:
        path.parent.mkdir(parents=True, exist_ok=True)
        tmp = path.with_suffix(path.suffix + ".tmp")
        tmp.write_text(self.to_json())
        tmp.replace(path)


def _flatten_union(tp) -> list:
    origin = get_origin(tp)
    if origin is typing.Annotated:
        return _flatten_union(get_args(tp)[0])
    if origin in (Union, types.UnionType):
        out = []
        for a in get_args(tp):
            out.extend(_flatten_union(a))
        return out
    return [tp]


def deep_merge(base: dict, other: dict) -> dict:
    out = dict(base)
    for k, v in other.items():
        if isinstance(v, dict) and isinstance(out.get(k), dict):
            out[k] = deep_merge(out[k], v)
        else:
            out[k] = v
    return out


def load_file(path: str | Path) -> dict:
    p = Path(path)
    if p.suffix == ".json":
        return json.loads(p.read_text())
    with open(p, "rb") as f:
        return tomllib.load(f)


def _strip_optional(tp):
    origin = get_origin(tp)
    if origin is typing.Annotated:
        return _strip_optional(get_args(tp)[0])
    if origin in (Union, types.UnionType):
        args = [a for a in get_args(tp) if a is not type(None)]
        return args
    return [tp]


def _field_type_candidates(model: type[BaseModel], name: str) -> list:
    fld = model.model_fields.get(name)
    if fld is None:
        return []
    out = []
    for a in _strip_optional(fld.annotation):
        out.extend(_strip_optional(a) if get_origin(a) is not None else [a])
    return out


def _resolve_path_types(model: type[BaseModel], parts: list[str], data: dict | None = None) -> list:
    """Types that the dotted path may have; follows sub-models (and union members, using the
    ``type`` discriminator found in ``data`` when present)."""
    cands: list = [model]
    cur_data: Any = data
    for i, part in enumerate(parts):
        nxt = []
        for c in cands:
            if isinstance(c, type) and issubclass(c, BaseModel):
                sub = _field_type_candidates(c, part)
                nxt.extend(sub)
        cur_data = cur_data.get(part) if isinstance(cur_data, dict) else None
        if isinstance(cur_data, dict) and "type" in cur_data:
            filtered = []
            for c in nxt:
                if isinstance(c, type) and issubclass(c, BaseModel) and "type" in c.model_fields:
                    if cur_data["type"] in get_args(c.model_fields["type"].annotation):
                        filtered.append(c)
            if filtered:
                nxt = filtered
        cands = nxt
    return cands


def _is_bool_field(cands: list) -> bool:
    return any(c is bool for c in cands)


def _is_model_field(cands: list) -> bool:
    return any(isinstance(c, type) and issubclass(c, BaseModel) for c in cands)


def _parse_scalar(s: str) -> Any:
    if s == "None" or s == "null":
        return None
    low = s.lower()
    if low == "true":
        return True
    if low == "false":
        return False
    if s and (s[0] in "[{\"" or s[0].isdigit() or s[0] in "-+."):
        try:
            return json.loads(s)
        except Exception:
            pass
        try:
            return tomllib.loads(f"v = {s}")["v"]
        except Exception:
            pass
    return s


def _set_path(d: dict, parts: list[str], value: Any) -> None:
    cur = d
    for p in parts[:-1]:
        if not isinstance(cur.get(p), dict):
            cur[p] = {}
        cur = cur[p]
    cur[parts[-1]] = value


def parse_argv(model: type[T], argv: list[str]) -> dict:
    """Turns ``@ file.toml ... --a.b-c value ...`` into a nested dict for ``model``."""
    data: dict = {}
    i = 0
    flags: list[tuple[list[str], Any]] = []
    while i < len(argv):
        tok = argv[i]
        if tok == "@":
            i += 1
            if i >= len(argv):
                raise SystemExit("'@' must be followed by a config file path")
            data = deep_merge(data, load_file(argv[i]))
            i += 1
            continue
        if tok.startswith("@") and len(tok) > 1:
            data = deep_merge(data, load_file(tok[1:]))
            i += 1
            continue
        if not tok.startswith("--"):
            raise SystemExit(f"unexpected argument '{tok}' (flags look like --section.field value)")
        key = tok[2:]
        value_inline = None
        if "=" in key:
            key, value_inline = key.split("=", 1)
        negated = False
        if key.startswith("no-"):
            negated = True
            key = key[3:]
        parts = [p.replace("-", "_") for p in key.split(".")]
        nxt = argv[i + 1] if i + 1 < len(argv) else None
        has_value = value_inline is not None or (nxt is not None and not nxt.startswith("--") and nxt != "@"
                                                 and not nxt.startswith("@"))
        # negative numbers look like flags; accept them as values
        if value_inline is None and nxt is not None and nxt.startswith("-") and not nxt.startswith("--"):
            try:
                float(nxt)
                has_value = True
            except ValueError:
                pass
        if negated:
            flags.append((parts, ("__negate__",)))
            i += 1
            continue
        if has_value:
            raw = value_inline if value_inline is not None else nxt
            flags.append((parts, _parse_scalar(raw)))
            i += 1 if value_inline is not None else 2
        else:
            flags.append((parts, ("__bare__",)))
            i += 1
    for parts, val in flags:
        cands = _resolve_path_types(model, parts, data)
        if val == ("__bare__",):
            if _is_bool_field(cands):
                _set_path(data, parts, True)
            elif _is_model_field(cands):
                cur = data
                ok = True
                for p in parts:
                    if not isinstance(cur, dict):
                        ok = False
                        break
                    cur = cur.get(p)
                if not (ok and isinstance(cur, dict)):
                    _set_path(data, parts, {})
            else:
                raise SystemExit(f"flag --{'.'.join(parts)} needs a value")
        elif val == ("__negate__",):
            if _is_bool_field(cands):
                _set_path(data, parts, False)
            else:
                _set_path(data, parts, None)
        else:
            _set_path(data, parts, val)
    return data


def _union_members(tp) -> list:
    out = []
    for a in _strip_optional(tp):
        if get_origin(a) in (Union, types.UnionType, typing.Annotated):
            out.extend(_union_members(a))
        else:
            out.append(a)
    return out


def inject_union_defaults(model: type[BaseModel], data: Any, recurse: bool = True) -> Any:
    """A partially specified discriminated-union block (``--optim.lr 1e-5`` without
    ``optim.type``) keeps the ``type`` of the field's default value."""
    if not isinstance(data, dict):
        return data
    for name, fld in model.model_fields.items():
        if name not in data or not isinstance(data[name], dict):
            continue
        members = [m for m in _union_members(fld.annotation) if isinstance(m, type) and issubclass(m, BaseModel)]
        if not members:
            continue
        sub = data[name] = dict(data[name])
        target = None
        if len(members) == 1:
            target = members[0]
        else:
            tagged = [m for m in members if "type" in m.model_fields]
            if "type" not in sub and tagged:
                default = fld.default if fld.default is not None else None
                if default is None and fld.default_factory is not None:
                    try:
                        default = fld.default_factory()
                    except Exception:
                        default = None
                if isinstance(default, BaseModel) and hasattr(default, "type"):
                    sub["type"] = default.type
                elif len(tagged) == len(members):
                    sub["type"] = get_args(tagged[0].model_fields["type"].annotation)[0]
            if "type" in sub:
                for m in tagged:
                    if sub["type"] in get_args(m.model_fields["type"].annotation):
                        target = m
                        break
            elif len(members) > 0 and not tagged:
                target = members[0]
        if target is not None and recurse:
            inject_union_defaults(target, sub)
    return data


def cli(model: type[T], argv: list[str] | None = None) -> T:
    """Parse the command line (``sys.argv[1:]`` by default) into ``model``."""
    argv = list(sys.argv[1:] if argv is None else argv)
    argv = [a for a in argv if a != "--dry-run"] if "dry_run" not in model.model_fields else argv
    data = parse_argv(model, argv)
    data = inject_union_defaults(model, data)
    return model.model_validate(data)
