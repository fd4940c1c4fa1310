"""Process-wide configuration object and its ``--<section>.<field>`` command line.

Behaviour follows pymllm/configs/global_config.py:27-79,173-351: one
singleton with the sections ``server``, ``model`` and ``quantization``; every
scalar dataclass field becomes an option named ``--<section>.<field>``; booleans
may be given bare (true) or with a value; only options that were actually typed
override the current values; the server section is rebuilt through its
constructor so validation runs again; ``model_path`` is mirrored between the
``server`` and ``model`` sections.
"""

from __future__ import annotations

import argparse
import dataclasses
import types
import typing
from pathlib import Path
from typing import Any, Callable, Iterator, Literal, Optional, Sequence, Union

from .model_config import ModelConfig
from .quantization_config import QuantizationConfig
from .server_config import ServerConfig

_SECTIONS = ("server", "model", "quantization")
_TRUE = frozenset({"1", "true", "t", "yes", "y", "on"})
_FALSE = frozenset({"0", "false", "f", "no", "n", "off"})


class GlobalConfig:
    """Singleton holding the three config sections."""

    _instance: Optional["GlobalConfig"] = None

    def __new__(cls) -> "GlobalConfig":
        if cls._instance is None:
            inst = super().__new__(cls)
            inst.server = ServerConfig(model_path=None)
            inst.model = ModelConfig()
            inst.quantization = QuantizationConfig()
            inst._initialized = True
            cls._instance = inst
        return cls._instance

    @classmethod
    def get_instance(cls) -> "GlobalConfig":
        return cls()

    @classmethod
    def reset(cls) -> None:
        """Drop the singleton so the next access starts from defaults (tests)."""
        cls._instance = None

    def __repr__(self) -> str:
        return (
            f"GlobalConfig(server={self.server!r}, model={self.model!r}, "
            f"quantization={self.quantization!r})"
        )


def get_global_config() -> GlobalConfig:
    return GlobalConfig.get_instance()


def _parse_bool(value: Any) -> bool:
    if isinstance(value, bool):
        return value
    if value is None:
        return True
    text = str(value).strip().lower()
    if text in _TRUE:
        return True
    if text in _FALSE:
        return False
    raise argparse.ArgumentTypeError(
        f"Invalid boolean value: {value!r}. Expected one of true/false, 1/0, yes/no."
    )


def _strip_optional(tp: Any) -> Any:
    if typing.get_origin(tp) in (Union, types.UnionType):
        rest = [a for a in typing.get_args(tp) if a is not type(None)]
        if len(rest) == 1:
            return rest[0]
    return tp


@dataclasses.dataclass
class _OptionSpec:
    section: str
    name: str
    kind: str  # "bool" | "scalar"
    convert: Optional[Callable[[str], Any]]
    choices: Optional[list]
    default: Any

    @property
    def flag(self) -> str:
        return f"--{self.section}.{self.name}"

    @property
    def dest(self) -> str:
        return f"{self.section}__{self.name}"


def _iter_option_specs(cfg: GlobalConfig) -> Iterator[_OptionSpec]:
    """Yield one spec per CLI-representable field; skip dicts, lists, handles."""
    for section in _SECTIONS:
        obj = getattr(cfg, section)
        hints = typing.get_type_hints(type(obj))
        for f in dataclasses.fields(obj):
            if f.name.startswith("_"):
                continue
            tp = _strip_optional(hints.get(f.name, f.type))
            default = getattr(obj, f.name)
            if tp is bool:
                yield _OptionSpec(section, f.name, "bool", _parse_bool, None, default)
            elif typing.get_origin(tp) is Literal:
                values = list(typing.get_args(tp))
                yield _OptionSpec(section, f.name, "scalar", type(values[0]), values, default)
            elif tp in (str, int, float, Path):
                yield _OptionSpec(section, f.name, "scalar", tp, None, default)


def make_args(parser: Optional[argparse.ArgumentParser] = None) -> argparse.ArgumentParser:
    """Add every ``--<section>.<field>`` option to ``parser`` (created if None).

    Defaults are suppressed so that :func:`read_args` can tell typed options from
    untouched ones.
    """
    if parser is None:
        parser = argparse.ArgumentParser(
            prog="mllm_b200", description="GlobalConfig options of mllm_b200."
        )
    groups: dict[str, Any] = {}
    for spec in _iter_option_specs(GlobalConfig.get_instance()):
        group = groups.get(spec.section)
        if group is None:
            group = groups[spec.section] = parser.add_argument_group(
                f"{spec.section} config", f"Fields of GlobalConfig.{spec.section}."
            )
        shown = "None" if spec.default is None else str(spec.default)
        if spec.kind == "bool":
            group.add_argument(
                spec.flag, dest=spec.dest, nargs="?", const=True, type=_parse_bool,
                default=argparse.SUPPRESS,
                help=f"bool, default {shown}; bare flag means true.",
            )
        else:
            extra = {"choices": spec.choices} if spec.choices is not None else {}
            group.add_argument(
                spec.flag, dest=spec.dest, type=spec.convert, default=argparse.SUPPRESS,
                help=f"default {shown}.", **extra,
            )
    return parser


def read_args(
    argv: Optional[Sequence[str]] = None,
    parser: Optional[argparse.ArgumentParser] = None,
) -> GlobalConfig:
    """Parse ``argv`` and apply the typed options onto the singleton."""
    if parser is None:
        parser = make_args()
    typed = vars(parser.parse_args(argv))
    cfg = GlobalConfig.get_instance()

    per_section: dict[str, dict[str, Any]] = {s: {} for s in _SECTIONS}
    for key, value in typed.items():
        section, sep, name = key.partition("__")
        if sep and section in per_section:
            per_section[section][name] = value

    if per_section["server"]:
        current = {f.name: getattr(cfg.server, f.name) for f in dataclasses.fields(cfg.server)}
        if "radix_cache_page_size" in per_section["server"] and "page_size" not in per_section["server"]:
            current["page_size"] = None
        current.update(per_section["server"])
        cfg.server = ServerConfig(**current)
    for section in ("model", "quantization"):
        for name, value in per_section[section].items():
            setattr(getattr(cfg, section), name, value)

    server_path_typed = "model_path" in per_section["server"]
    model_path_typed = "model_path" in per_section["model"]
    if server_path_typed and not model_path_typed:
        cfg.model.model_path = cfg.server.model_path
    elif model_path_typed and not server_path_typed:
        cfg.server.model_path = cfg.model.model_path
    return cfg
