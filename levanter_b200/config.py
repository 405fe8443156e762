"""Dataclass configuration: YAML files + dotted command-line overrides + ``type:``-selected plugin classes.

Covers what the reference gets from ``draccus`` plus its own ``levanter.config.main`` wrapper
(src/levanter/config.py:79-169): ``--config_path/--config/--configs``, bare config names resolved in a
config directory with ``.yaml``/``.yml`` suffixes, URL configs through fsspec, concatenation of several
config files, ``!include`` of other YAML files, and the scalar codecs for mixed-precision policies
(``"p=f32,c=bfloat16"``), durations (``"5m"``), dtypes and remat policies (src/levanter/config.py:27-70).
"""
from __future__ import annotations

import dataclasses
import enum
import functools
import inspect
import pathlib
import os
import sys
import tempfile
import typing
from dataclasses import MISSING, fields, is_dataclass
from datetime import timedelta
from typing import Any, Callable, ClassVar, Dict, List, Optional, Type, TypeVar, Union, get_args, get_origin

import torch
import yaml

from .utils.datetime_utils import encode_timedelta, parse_timedelta

T = TypeVar("T")
DEFAULT_CONFIG_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "config")


class ConfigError(ValueError):
    pass


class UnknownChoiceError(ConfigError, KeyError):
    """A ``type:`` name that no class is registered under (a ``KeyError`` too: a registry is looked up like a mapping)."""

    def __str__(self) -> str:  # KeyError would print the repr of the message
        return str(self.args[0]) if self.args else ""


# --------------------------------------------------------------------------- plugin registries
class ChoiceRegistry:
    """Base for config classes selected by a ``type:`` key (model, optimizer, tracker, rope, ...).

    Each direct subclass of ``ChoiceRegistry`` owns one registry; implementations register with
    ``@Base.register_subclass("name")``.
    """

    _choice_registry: ClassVar[Dict[str, type]]
    _registry_root: ClassVar[Optional[type]] = None

    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        if ChoiceRegistry in cls.__bases__:
            cls._choice_registry = {}
            cls._registry_root = cls

    @classmethod
    def register_subclass(cls, name: str):
        def deco(sub):
            cls._registry_root._choice_registry[name] = sub
            sub._choice_name = name
            return sub

        return deco

    @classmethod
    def get_choice_class(cls, name: str) -> type:
        reg = cls._registry_root._choice_registry
        if name not in reg:
            raise UnknownChoiceError(f"unknown {cls._registry_root.__name__} type {name!r}; known: {sorted(reg)}")
        return reg[name]

    @classmethod
    def get_known_choices(cls) -> Dict[str, type]:
        return dict(cls._registry_root._choice_registry)

    @classmethod
    def default_choice_name(cls) -> Optional[str]:
        return None

    @classmethod
    def get_choice_name(cls, sub: type) -> str:
        for k, v in cls._registry_root._choice_registry.items():
            if v is sub:
                return k
        raise ConfigError(f"{sub} is not registered")


def _is_registry(tp) -> bool:
    return inspect.isclass(tp) and issubclass(tp, ChoiceRegistry) and tp._registry_root is not None


# --------------------------------------------------------------------------- mixed precision policy
_DTYPES = {
    "f32": torch.float32, "float32": torch.float32, "fp32": torch.float32, "float": torch.float32, "full": torch.float32,
    "bf16": torch.bfloat16, "bfloat16": torch.bfloat16,
    "f16": torch.float16, "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
    "f64": torch.float64, "float64": torch.float64,
    "int32": torch.int32, "int64": torch.int64, "int8": torch.int8, "uint8": torch.uint8, "bool": torch.bool,
    "float8_e4m3fn": torch.float8_e4m3fn, "float8_e5m2": torch.float8_e5m2,
}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    key = str(name).replace("torch.", "").replace("jnp.", "").lower()
    if key not in _DTYPES:
        raise ConfigError(f"unknown dtype {name!r}")
    return _DTYPES[key]


def dtype_name(dt: torch.dtype) -> str:
    return str(dt).replace("torch.", "")


@dataclasses.dataclass(frozen=True)
class Policy:
    """Mixed-precision policy with jmp's string grammar (``"bfloat16"``, ``"p=f32,c=bfloat16"``,
    ``"compute=bfloat16,params=float32,output=bfloat16"``).  Trainable parameters live in
    ``param_dtype``; the loss casts the model to ``compute_dtype`` on entry; outputs are cast to
    ``output_dtype`` (src/levanter/trainer_state.py:216-226, src/levanter/trainer.py:208-210)."""

    param_dtype: torch.dtype = torch.float32
    compute_dtype: torch.dtype = torch.float32
    output_dtype: torch.dtype = torch.float32

    @staticmethod
    def parse(s: Union[str, "Policy"]) -> "Policy":
        if isinstance(s, Policy):
            return s
        s = str(s).strip()
        if "=" not in s:
            dt = parse_dtype(s)
            return Policy(dt, dt, dt)
        param = compute = output = None
        for part in s.split(","):
            k, v = part.split("=")
            k = k.strip()
            dt = parse_dtype(v.strip())
            if k in ("p", "params", "param"):
                param = dt
            elif k in ("c", "compute"):
                compute = dt
            elif k in ("o", "output"):
                output = dt
            else:
                raise ConfigError(f"unknown key {k!r} in precision policy {s!r}")
        param = param or torch.float32
        compute = compute or param
        output = output or compute
        return Policy(param, compute, output)

    def __str__(self):
        return (f"compute={dtype_name(self.compute_dtype)},params={dtype_name(self.param_dtype)},"
                f"output={dtype_name(self.output_dtype)}")

    def cast_to_compute(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(self.compute_dtype) if t.is_floating_point() else t

    def cast_to_param(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(self.param_dtype) if t.is_floating_point() else t

    def cast_to_output(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(self.output_dtype) if t.is_floating_point() else t


# --------------------------------------------------------------------------- custom codecs
_DECODERS: Dict[type, Callable[[Any], Any]] = {
    timedelta: lambda v: v if isinstance(v, timedelta) else parse_timedelta(str(v)),
    torch.dtype: parse_dtype,
    Policy: Policy.parse,
    pathlib.Path: lambda v: pathlib.Path(str(v)),
}
_ENCODERS: Dict[type, Callable[[Any], Any]] = {
    timedelta: encode_timedelta,
    torch.dtype: dtype_name,
    Policy: str,
    pathlib.Path: str,
}


def register_codec(tp: type, decoder: Callable[[Any], Any], encoder: Callable[[Any], Any]) -> None:
    _DECODERS[tp] = decoder
    _ENCODERS[tp] = encoder


# --------------------------------------------------------------------------- YAML with !include
class _IncludeLoader(yaml.SafeLoader):
    def __init__(self, stream, base_dir: str):
        self._base_dir = base_dir
        super().__init__(stream)


def _include(loader: _IncludeLoader, node):
    rel = loader.construct_scalar(node)
    path = rel if os.path.isabs(rel) or "://" in rel else os.path.join(loader._base_dir, rel)
    return load_yaml(path)


_IncludeLoader.add_constructor("!include", _include)
# YAML 1.1 reads "1E-3" (no dot) as a string; accept it as a float like the reference's loader does.
import re as _re

_IncludeLoader.add_implicit_resolver(
    "tag:yaml.org,2002:float",
    _re.compile(r"^[-+]?(?:[0-9][0-9_]*)(?:\.[0-9_]*)?[eE][-+]?[0-9]+$"),
    list("-+0123456789"),
)


def _read_text(path: str) -> str:
    if "://" in path:
        import fsspec

        with fsspec.open(path, "r") as f:
            return f.read()
    with open(path, "r") as f:
        return f.read()


def load_yaml(path: str) -> Any:
    text = _read_text(path)
    base = os.path.dirname(path)
    loader = _IncludeLoader(text, base)
    try:
        return loader.get_single_data()
    finally:
        loader.dispose()


# --------------------------------------------------------------------------- decoding
def _type_hints(cls) -> Dict[str, Any]:
    try:
        return typing.get_type_hints(cls)
    except Exception:
        # one unresolvable forward reference must not turn every other field into a string: resolve field by field
        import sys

        out: Dict[str, Any] = {}
        for klass in reversed(cls.__mro__):
            ns = dict(vars(sys.modules.get(klass.__module__, typing)))
            ns.update(vars(typing))
            for name, ann in getattr(klass, "__annotations__", {}).items():
                if isinstance(ann, str):
                    try:
                        ann = eval(ann, ns)  # noqa: S307 - annotations of our own config classes
                    except Exception:
                        ann = Any
                out[name] = ann
        return out


def _coerce_scalar(tp, value, path):
    if tp is bool:
        if isinstance(value, bool):
            return value
        if isinstance(value, str) and value.lower() in ("true", "false", "1", "0", "yes", "no"):
            return value.lower() in ("true", "1", "yes")
        raise ConfigError(f"{path}: expected bool, got {value!r}")
    if tp is int:
        if isinstance(value, bool):
            raise ConfigError(f"{path}: expected int, got bool")
        if isinstance(value, int):
            return value
        if isinstance(value, float) and value.is_integer():
            return int(value)
        if isinstance(value, str):
            try:
                return int(value)
            except ValueError:
                try:
                    f = float(value)  # "1e3" style integers
                except ValueError:
                    f = None
                if f is not None and f.is_integer():
                    return int(f)
        raise ConfigError(f"{path}: expected int, got {value!r}")
    if tp is float:
        if isinstance(value, bool):
            raise ConfigError(f"{path}: expected float, got bool")
        if isinstance(value, (int, float)):
            return float(value)
        if isinstance(value, str):
            try:
                return float(value)
            except ValueError:
                pass
        raise ConfigError(f"{path}: expected float, got {value!r}")
    if tp is str:
        if isinstance(value, (dict, list)):
            raise ConfigError(f"{path}: expected str, got {type(value).__name__}")
        return str(value)
    raise ConfigError(f"{path}: unsupported scalar type {tp}")


def decode(tp, value, path: str = "<root>"):
    """Turn parsed YAML (``dict``/``list``/scalars) into an instance of ``tp``."""
    if tp is Any or tp is inspect.Parameter.empty or isinstance(tp, TypeVar):
        return value
    origin = get_origin(tp)
    if origin is Union or (hasattr(__import__("types"), "UnionType") and isinstance(tp, __import__("types").UnionType)):
        args = get_args(tp)
        if value is None and type(None) in args:
            return None
        errors = []
        # exact-type scalars first so "1" vs 1 are not confused, then structural attempts in order
        for a in args:
            if a in (int, float, bool, str) and type(value) is a:
                return value
        for a in args:
            if a is type(None):
                continue
            try:
                return decode(a, value, path)
            except (ConfigError, TypeError, ValueError, KeyError) as e:
                errors.append(f"{a}: {e}")
        raise ConfigError(f"{path}: value {value!r} fits no member of {tp}:\n  " + "\n  ".join(errors))
    if origin is typing.Literal:
        if value in get_args(tp):
            return value
        raise ConfigError(f"{path}: {value!r} not in {get_args(tp)}")
    if origin in (list, typing.List, typing.Sequence, typing.Iterable) or tp in (list, typing.List):
        if isinstance(value, str) and path.startswith("--"):
            value = yaml.safe_load(value)
        if not isinstance(value, (list, tuple)):
            raise ConfigError(f"{path}: expected a list, got {value!r}")
        (elem,) = get_args(tp) or (Any,)
        return [decode(elem, v, f"{path}[{i}]") for i, v in enumerate(value)]
    if origin in (tuple, typing.Tuple) or tp is tuple:
        if not isinstance(value, (list, tuple)):
            raise ConfigError(f"{path}: expected a sequence, got {value!r}")
        args = get_args(tp)
        if not args:
            return tuple(value)
        if len(args) == 2 and args[1] is Ellipsis:
            return tuple(decode(args[0], v, f"{path}[{i}]") for i, v in enumerate(value))
        if len(args) != len(value):
            raise ConfigError(f"{path}: expected {len(args)} items")
        return tuple(decode(a, v, f"{path}[{i}]") for i, (a, v) in enumerate(zip(args, value)))
    if origin in (dict, typing.Dict, typing.Mapping) or tp is dict:
        if value is None:
            return {}
        if not isinstance(value, dict):
            raise ConfigError(f"{path}: expected a mapping, got {value!r}")
        args = get_args(tp)
        kt, vt = args if len(args) == 2 else (Any, Any)
        return {decode(kt, k, f"{path}.{k}"): decode(vt, v, f"{path}.{k}") for k, v in value.items()}
    if origin in (set, frozenset, typing.Set, typing.FrozenSet, typing.AbstractSet):
        (elem,) = get_args(tp) or (Any,)
        if not isinstance(value, (list, tuple, set)):
            value = [value]
        return set(decode(elem, v, path) for v in value)
    if inspect.isclass(tp):
        if tp in _DECODERS:
            if isinstance(value, tp):
                return value
            return _DECODERS[tp](value)
        for base, dec in _DECODERS.items():
            if issubclass(tp, base):
                return dec(value)
        if issubclass(tp, enum.Enum):
            if isinstance(value, tp):
                return value
            try:
                return tp[value] if isinstance(value, str) and value in tp.__members__ else tp(value)
            except Exception:
                raise ConfigError(f"{path}: {value!r} is not a member of {tp.__name__}")
        if hasattr(tp, "from_config_value") and not isinstance(value, dict):
            return tp.from_config_value(value)
        if is_dataclass(tp) or _is_registry(tp):
            return _decode_dataclass(tp, value, path)
        if tp in (int, float, bool, str):
            return _coerce_scalar(tp, value, path)
        if isinstance(value, tp):
            return value
    raise ConfigError(f"{path}: cannot decode {value!r} as {tp}")


def _decode_dataclass(tp, value, path):
    if isinstance(value, tp) and not isinstance(value, dict):
        return value
    if value is None:
        value = {}
    if not isinstance(value, dict):
        raise ConfigError(f"{path}: expected a mapping for {tp.__name__}, got {value!r}")
    value = dict(value)
    cls = tp
    if _is_registry(tp):
        name = value.pop("type", None)
        if name is None:
            if getattr(tp, "_choice_name", None) is not None and is_dataclass(tp) and tp is not tp._registry_root:
                name = tp._choice_name
            else:
                name = tp.default_choice_name()
        if name is None:
            if is_dataclass(tp) and not inspect.isabstract(tp):
                cls = tp
            else:
                raise ConfigError(f"{path}: missing 'type' (one of {sorted(tp.get_known_choices())})")
        else:
            cls = tp.get_choice_class(name)
            if not (inspect.isclass(cls) and issubclass(cls, tp)) and tp is not tp._registry_root:
                raise ConfigError(f"{path}: type {name!r} is not a {tp.__name__}")
    if not is_dataclass(cls):
        raise ConfigError(f"{path}: {cls} is not a dataclass")
    hints = _type_hints(cls)
    kwargs = {}
    names = {f.name for f in fields(cls) if f.init}
    for k in list(value.keys()):
        if k not in names:
            raise ConfigError(f"{path}: unknown key {k!r} for {cls.__name__} (known: {sorted(names)})")
    for f in fields(cls):
        if not f.init:
            continue
        if f.name in value:
            kwargs[f.name] = decode(hints.get(f.name, Any), value[f.name], f"{path}.{f.name}")
        elif f.default is MISSING and f.default_factory is MISSING:
            ftp = hints.get(f.name, Any)
            if (inspect.isclass(ftp) and (is_dataclass(ftp) or _is_registry(ftp))):
                kwargs[f.name] = decode(ftp, {}, f"{path}.{f.name}")
            else:
                raise ConfigError(f"{path}: missing required key {f.name!r} for {cls.__name__}")
    return cls(**kwargs)


# --------------------------------------------------------------------------- encoding
def encode(obj) -> Any:
    """Inverse of :func:`decode`: a YAML/JSON-able tree."""
    if isinstance(obj, enum.Enum):  # before the scalar test: ``class E(str, Enum)`` members are also ``str``
        return obj.name if not isinstance(obj.value, str) else str(obj.value)
    if obj is None or isinstance(obj, (bool, int, float, str)):
        return obj
    for tp, enc in _ENCODERS.items():
        if isinstance(obj, tp):
            return enc(obj)
    if isinstance(obj, enum.Enum):
        return obj.name if not isinstance(obj.value, str) else obj.value
    if is_dataclass(obj) and not isinstance(obj, type):
        out = {}
        cls = type(obj)
        if _is_registry(cls) and getattr(cls, "_choice_name", None) is not None:
            out["type"] = cls._choice_name
        for f in fields(obj):
            if f.init:
                out[f.name] = encode(getattr(obj, f.name))
        return out
    if isinstance(obj, dict):
        return {str(k): encode(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple, set, frozenset)):
        return [encode(v) for v in obj]
    if hasattr(obj, "to_config_value"):
        return obj.to_config_value()
    return str(obj)


def to_yaml(obj) -> str:
    return yaml.safe_dump(encode(obj), sort_keys=False)


# --------------------------------------------------------------------------- command line
def _set_dotted(tree: dict, dotted: str, value):
    keys = dotted.split(".")
    cur = tree
    for k in keys[:-1]:
        nxt = cur.get(k)
        if not isinstance(nxt, dict):
            nxt = {}
            cur[k] = nxt
        cur = nxt
    cur[keys[-1]] = value


def _parse_cli_value(s: str):
    try:
        v = yaml.load(s, Loader=_make_plain_loader())
    except yaml.YAMLError:
        return s
    return v


def _make_plain_loader():
    class L(yaml.SafeLoader):
        pass

    L.add_implicit_resolver(
        "tag:yaml.org,2002:float",
        _re.compile(r"^[-+]?(?:[0-9][0-9_]*)(?:\.[0-9_]*)?[eE][-+]?[0-9]+$"),
        list("-+0123456789"),
    )
    return L


def _deep_merge(a: dict, b: dict) -> dict:
    out = dict(a)
    for k, v in b.items():
        if isinstance(v, dict) and isinstance(out.get(k), dict):
            out[k] = _deep_merge(out[k], v)
        else:
            out[k] = v
    return out


def split_config_args(args: List[str]):
    """Pull ``--config_path X`` / ``--config X`` / ``--configs A B ...`` out of ``args``.

    Returns ``(list_of_config_paths, remaining_args)`` (src/levanter/config.py:116-169)."""
    paths: List[str] = []
    rest: List[str] = []
    i = 0
    while i < len(args):
        a = args[i]
        key, eq, val = a.partition("=")
        if key in ("--config_path", "--config"):
            if eq:
                paths.append(val)
                i += 1
            else:
                if i + 1 >= len(args):
                    raise ConfigError(f"{key} needs a value")
                paths.append(args[i + 1])
                i += 2
        elif key == "--configs":
            i += 1
            if eq:
                paths.append(val)
            while i < len(args) and not args[i].startswith("--"):
                paths.append(args[i])
                i += 1
        else:
            rest.append(a)
            i += 1
    return paths, rest


def resolve_config_path(path: str, config_dir: Optional[str] = DEFAULT_CONFIG_DIR) -> str:
    if "://" in path:
        import fsspec

        fd, tmp = tempfile.mkstemp(suffix=".yaml")
        with fsspec.open(path, "r") as f, os.fdopen(fd, "w") as out:
            out.write(f.read())
        return tmp
    cands = [path, f"{path}.yaml", f"{path}.yml"]
    if config_dir is not None:
        cands += [os.path.join(config_dir, c) for c in list(cands)]
    for c in cands:
        if os.path.exists(c):
            return c
    raise ConfigError(f"config {path!r} not found (looked at {cands})")


def parse_overrides(args: List[str]) -> dict:
    tree: dict = {}
    i = 0
    while i < len(args):
        a = args[i]
        if not a.startswith("--"):
            raise ConfigError(f"unexpected argument {a!r}")
        key, eq, val = a[2:].partition("=")
        if eq:
            _set_dotted(tree, key, _parse_cli_value(val))
            i += 1
        else:
            vals = []
            i += 1
            while i < len(args) and not (args[i].startswith("--") and not _looks_negative_number(args[i])):
                vals.append(args[i])
                i += 1
            if not vals:
                _set_dotted(tree, key, True)
            elif len(vals) == 1:
                _set_dotted(tree, key, _parse_cli_value(vals[0]))
            else:
                _set_dotted(tree, key, [_parse_cli_value(v) for v in vals])
    return tree


def _looks_negative_number(s: str) -> bool:
    try:
        float(s)
        return True
    except ValueError:
        return False


def parse(config_class: Type[T], config_path: Union[None, str, List[str]] = None, args: Optional[List[str]] = None,
          config_dir: Optional[str] = DEFAULT_CONFIG_DIR) -> T:
    """Build ``config_class`` from YAML file(s) and ``--dotted.key value`` overrides."""
    tree: dict = {}
    paths = [] if config_path is None else ([config_path] if isinstance(config_path, str) else list(config_path))
    for p in paths:
        data = load_yaml(resolve_config_path(p, config_dir)) or {}
        if not isinstance(data, dict):
            raise ConfigError(f"{p}: top level of a config must be a mapping")
        tree = _deep_merge(tree, data)
    if args:
        tree = _deep_merge(tree, parse_overrides(list(args)))
    return decode(config_class, tree, "<config>")


def main(fn=None, *, args: Optional[List[str]] = None, config_dir: Optional[str] = DEFAULT_CONFIG_DIR):
    """Decorator: ``@levanter_b200.config.main`` on ``def main(config: SomeConfig)`` parses the process
    arguments into ``SomeConfig`` and calls the function (src/levanter/config.py:79-113)."""
    if fn is None:
        return functools.partial(main, args=args, config_dir=config_dir)
    cmd_args = args

    @functools.wraps(fn)
    def wrapper(*a, **kw):
        spec = inspect.getfullargspec(fn)
        hints = typing.get_type_hints(fn)
        cfg_type = hints[spec.args[0]]
        if a and isinstance(a[0], cfg_type):
            return fn(*a, **kw)  # called from Python with a ready configuration: nothing to parse
        argv = list(sys.argv[1:] if cmd_args is None else cmd_args)
        paths, rest = split_config_args(argv)
        cfg = parse(cfg_type, paths, rest, config_dir)
        return fn(cfg, *a, **kw)

    return wrapper
