"""What every architecture's configuration shares: the error type, typed readers of
``config.json`` keys, and the reading of a model folder's JSON files."""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional


class ConfigError(ValueError):
    pass


def need_int(d: Dict[str, Any], key: str, default: Optional[int] = None, minimum: int = 1) -> int:
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    if isinstance(v, bool) or not isinstance(v, int):
        if isinstance(v, float) and v == int(v):
            v = int(v)
        else:
            raise ConfigError(f"config.json: '{key}' must be an integer, found {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: '{key}' must be >= {minimum}, found {v}")
    return v


def need_float(d: Dict[str, Any], key: str, default: Optional[float] = None) -> float:
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: '{key}' must be a number, found {v!r}")
    return float(v)


def token_id_list(v: Any, key: str, where: str = "config.json") -> tuple:
    """An id, a list of ids, or nothing."""
    if v is None:
        return ()
    if isinstance(v, int) and not isinstance(v, bool):
        return (v,)
    if isinstance(v, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in v):
        return tuple(v)
    raise ConfigError(f"{where}: {key} must be an integer or a list of integers, found {v!r}")


def _load_json_object(path: str) -> Dict[str, Any]:
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: the top level must be an object")
    return d


def load_config_dict(model_dir: str) -> Dict[str, Any]:
    """``config.json`` of a model folder.  If the folder also has a ``generation_config.json`` with an
    ``eos_token_id``, those ids are added to ``config.json``'s: generation stops at any of them (the
    reference stops at the end-of-sequence id and at every end-of-turn marker its vocabulary has,
    src/tokenizer.cpp:68-77)."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json in the model folder")
    d = _load_json_object(path)
    gpath = os.path.join(model_dir, "generation_config.json")
    if os.path.isfile(gpath):
        g = _load_json_object(gpath)
        more = token_id_list(g.get("eos_token_id"), "eos_token_id", "generation_config.json")
        if more:
            have = token_id_list(d.get("eos_token_id"), "eos_token_id")
            ids = list(have) + [i for i in more if i not in have]
            d = dict(d)
            d["eos_token_id"] = ids if len(ids) > 1 else ids[0]
    return d
