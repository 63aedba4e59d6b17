"""The one registry from an architecture's name to its configuration class.

QStream's converter keeps a dict `model_type -> arch` and falls back to llama for
unknown types (tools/convert_hf.py:1540-1569).  Here `architectures[0]` of
config.json (or `model_type`, as an alias) is looked up; an unknown name is an
error, never a silent fallback.

A configuration class offers `from_dict(dict)`, `to_dict()`, `model_spec()` and the
attributes `architecture` and `model_type`; that is all the rest of the library
asks of an architecture.
"""
from __future__ import annotations

import json
from pathlib import Path

from ..errors import QsError, QStreamError

_ARCHITECTURES: dict[str, type] = {}


def register_architecture(config_cls, *aliases: str) -> None:
    """Make `config_cls` the configuration of `config_cls.architecture` (and of the
    aliases, usually its `model_type`)."""
    for name in (config_cls.architecture, *aliases):
        _ARCHITECTURES[name] = config_cls


def architecture_names() -> list[str]:
    return sorted(_ARCHITECTURES)


def config_class_for(name: str):
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise QStreamError(QsError.UNSUPPORTED_ARCH,
                           f"architecture '{name}' is not registered "
                           f"(known: {', '.join(architecture_names())})") from None


def config_from_dict(d: dict):
    archs = d.get("architectures") or []
    name = archs[0] if archs else d.get("model_type")
    if not name:
        raise QStreamError(QsError.INVALID_MODEL,
                           "config.json names no architecture ('architectures' or 'model_type')")
    return config_class_for(name).from_dict(d)


def load_config(folder):
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise QStreamError(QsError.FILE_NOT_FOUND, str(path))
    try:
        d = json.loads(path.read_text())
    except (ValueError, UnicodeDecodeError) as e:
        raise QStreamError(QsError.FILE_CORRUPTED, f"{path}: {e}") from None
    if not isinstance(d, dict):
        raise QStreamError(QsError.FILE_CORRUPTED, f"{path}: not a JSON object")
    return config_from_dict(d)
