"""Typed readers for config.json values.  Every error names the key
(the reference does the same: crates/thuban_model/src/config.rs:4-34)."""
from __future__ import annotations

from ..errors import ConfigError

_MISSING = object()


def _find(d, key, aliases):
    for k in (key, *aliases):
        if k in d and d[k] is not None:
            return k, d[k]
    return key, _MISSING


def get_int(d, key, default=_MISSING, aliases=(), minimum=None):
    k, v = _find(d, key, aliases)
    if v is _MISSING:
        if default is _MISSING:
            raise ConfigError(f"missing config field {key!r}")
        return default
    if isinstance(v, bool) or not isinstance(v, int):
        if isinstance(v, float) and v.is_integer():
            v = int(v)
        else:
            raise ConfigError(f"config field {k!r} must be an integer, got {v!r}")
    if minimum is not None and v < minimum:
        raise ConfigError(f"config field {k!r} must be >= {minimum}, got {v}")
    return v


def get_float(d, key, default=_MISSING, aliases=()):
    k, v = _find(d, key, aliases)
    if v is _MISSING:
        if default is _MISSING:
            raise ConfigError(f"missing config field {key!r}")
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config field {k!r} must be a number, got {v!r}")
    return float(v)


def get_bool(d, key, default=_MISSING, aliases=()):
    k, v = _find(d, key, aliases)
    if v is _MISSING:
        if default is _MISSING:
            raise ConfigError(f"missing config field {key!r}")
        return default
    if not isinstance(v, bool):
        raise ConfigError(f"config field {k!r} must be true or false, got {v!r}")
    return v


def get_str(d, key, default=_MISSING, aliases=()):
    k, v = _find(d, key, aliases)
    if v is _MISSING:
        if default is _MISSING:
            raise ConfigError(f"missing config field {key!r}")
        return default
    if not isinstance(v, str):
        raise ConfigError(f"config field {k!r} must be a string, got {v!r}")
    return v


def get_int_list(d, key, aliases=()):
    """int | list of int | null -> tuple (crates/thuban_model/src/config.rs:22-29)."""
    k, v = _find(d, key, aliases)
    if v is _MISSING:
        return ()
    if isinstance(v, int) and not isinstance(v, bool):
        return (v,)
    if isinstance(v, list) and all(isinstance(x, int) and not isinstance(x, bool) for x in v):
        return tuple(v)
    raise ConfigError(f"config field {k!r} must be an integer or a list of integers, got {v!r}")


def get_float_list(d, key, length=None, aliases=()):
    k, v = _find(d, key, aliases)
    if v is _MISSING:
        raise ConfigError(f"missing config field {key!r}")
    if not isinstance(v, list) or not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in v):
        raise ConfigError(f"config field {k!r} must be a list of numbers")
    if length is not None and len(v) != length:
        raise ConfigError(f"config field {k!r} must have {length} entries, got {len(v)}")
    return tuple(float(x) for x in v)
