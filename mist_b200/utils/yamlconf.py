"""A small YAML configuration composer with the subset of Hydra/OmegaConf semantics
that the analyze / exec / tune entry points rely on, so existing experiment YAMLs
keep working without either package installed:

* ``defaults:`` lists (``- _self_``, ``- group: option``, ``- /group/option``,
  ``- group: null``), composed depth-first; files marked ``# @package _global_`` (all of
  ours) merge at the root.
* ``${a.b.c}`` interpolation (``${hydra:runtime.cwd}`` resolves to the working directory).
* command-line overrides ``a.b=value``, ``+a.b=value`` (add), ``~a.b`` (delete) and the
  ``--config-name/-cn``, ``--config-path/-cp``, ``--config-dir/-cd`` flags.

The result is a :class:`Node`: a dict with attribute access, which is all the config
objects in :mod:`mist_b200.config` need (reference: benchmark/mist/configs/config.yaml:1-33
and the hydra.main decorators at benchmark/mist/analysis/run.py:197-202).
"""
from __future__ import annotations

import copy
import os
import re
import sys
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence

import yaml


class Node(dict):
    """dict with attribute access (missing attributes raise AttributeError)."""

    def __getattr__(self, key):
        try:
            return self[key]
        except KeyError as e:
            raise AttributeError(key) from e

    def __setattr__(self, key, value):
        self[key] = value

    def to_dict(self):
        return _to_plain(self)


def _to_node(obj):
    if isinstance(obj, dict):
        return Node({k: _to_node(v) for k, v in obj.items()})
    if isinstance(obj, list):
        return [_to_node(v) for v in obj]
    return obj


def _to_plain(obj):
    if isinstance(obj, dict):
        return {k: _to_plain(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_to_plain(v) for v in obj]
    return obj


def merge(dst: dict, src: dict) -> dict:
    """Recursive merge of ``src`` into ``dst`` (lists and scalars are replaced)."""
    for k, v in src.items():
        if isinstance(v, dict) and isinstance(dst.get(k), dict):
            merge(dst[k], v)
        else:
            dst[k] = copy.deepcopy(v)
    return dst


def _load_yaml(path: Path) -> dict:
    with open(path) as f:
        data = yaml.safe_load(f)
    return data or {}


def _find(config_dirs: Sequence[Path], rel: str) -> Path:
    rel = rel.lstrip("/")
    for d in config_dirs:
        for cand in (d / rel, d / (rel + ".yaml")):
            if cand.is_file():
                return cand
    raise FileNotFoundError(f"config '{rel}' not found under {[str(d) for d in config_dirs]}")


def _compose_file(path: Path, config_dirs: Sequence[Path], group_dir: str, overrides: Dict[str, str]) -> dict:
    raw = _load_yaml(path)
    defaults = raw.pop("defaults", None)
    if defaults is None:
        return raw
    out: dict = {}
    self_done = False
    for entry in defaults:
        if entry == "_self_":
            merge(out, raw)
            self_done = True
            continue
        if isinstance(entry, str):
            rel = entry if entry.startswith("/") else (f"{group_dir}/{entry}" if group_dir else entry)
            sub = _find(config_dirs, rel)
            merge(out, _compose_file(sub, config_dirs, os.path.dirname(rel.lstrip("/")), overrides))
            continue
        if isinstance(entry, dict):
            for group, option in entry.items():
                group = str(group)
                if group.startswith("override "):
                    group = group[len("override "):]
                option = overrides.get(group.lstrip("/"), option)
                if option is None or option == "null":
                    continue
                rel = f"{group}/{option}"
                sub = _find(config_dirs, rel)
                merge(out, _compose_file(sub, config_dirs, group.lstrip("/"), overrides))
    if not self_done:
        merge(out, raw)
    return out


_INTERP = re.compile(r"\$\{([^${}]+)\}")


def _lookup(root: dict, dotted: str):
    cur: Any = root
    for part in dotted.split("."):
        if isinstance(cur, list):
            cur = cur[int(part)]
        else:
            cur = cur[part]
    return cur


def _resolve_value(val, root, depth=0):
    if depth > 20:
        raise ValueError("interpolation cycle")
    if isinstance(val, str):
        m = _INTERP.fullmatch(val.strip())
        if m:  # whole-string interpolation keeps the referenced type
            return _resolve_value(_resolve_key(m.group(1), root), root, depth + 1)
        if _INTERP.search(val):
            return _INTERP.sub(lambda mm: str(_resolve_value(_resolve_key(mm.group(1), root), root, depth + 1)), val)
        return val
    if isinstance(val, dict):
        return {k: _resolve_value(v, root, depth) for k, v in val.items()}
    if isinstance(val, list):
        return [_resolve_value(v, root, depth) for v in val]
    return val


def _resolve_key(key: str, root):
    key = key.strip()
    if key.startswith("hydra:"):
        if key == "hydra:runtime.cwd":
            return os.getcwd()
        return ""
    if key.startswith("oc.env:"):
        name, _, default = key[len("oc.env:"):].partition(",")
        return os.environ.get(name.strip(), default.strip())
    return _lookup(root, key)


def resolve(cfg: dict) -> dict:
    return _resolve_value(cfg, cfg)


def _parse_scalar(text: str):
    try:
        return yaml.safe_load(text)
    except yaml.YAMLError:
        return text


def _set_dotted(cfg: dict, dotted: str, value, must_exist: bool):
    parts = dotted.split(".")
    cur = cfg
    for p in parts[:-1]:
        if p not in cur or not isinstance(cur[p], dict):
            if must_exist:
                raise KeyError(f"override '{dotted}': '{p}' does not exist (use +{dotted}=... to add)")
            cur[p] = {}
        cur = cur[p]
    if must_exist and parts[-1] not in cur:
        raise KeyError(f"override '{dotted}' does not exist (use +{dotted}=... to add)")
    cur[parts[-1]] = value


def compose(config_name: str, config_dirs: Sequence[os.PathLike], overrides: Optional[List[str]] = None,
            do_resolve: bool = True) -> Node:
    """Loads ``config_name`` from the first directory that has it and applies overrides."""
    dirs = [Path(d) for d in config_dirs]
    overrides = list(overrides or [])
    group_over: Dict[str, str] = {}
    value_over = []
    for ov in overrides:
        if ov.startswith("~"):
            value_over.append(("del", ov[1:], None))
            continue
        key, eq, val = ov.partition("=")
        if not eq:
            raise ValueError(f"cannot parse override '{ov}'")
        add = key.startswith("+")
        key = key.lstrip("+")
        # a bare group name selects a config-group option (experiment=..., model=...)
        if "." not in key and any((d / key).is_dir() for d in dirs) and not add:
            group_over[key] = val
        else:
            value_over.append(("add" if add else "set", key, _parse_scalar(val)))
    root_file = _find(dirs, config_name)
    cfg = _compose_file(root_file, dirs, "", group_over)
    for kind, key, val in value_over:
        if kind == "del":
            cur = cfg
            parts = key.split(".")
            for p in parts[:-1]:
                cur = cur[p]
            cur.pop(parts[-1], None)
        else:
            _set_dotted(cfg, key, val, must_exist=False)
    if do_resolve:
        cfg = resolve(cfg)
    return _to_node(cfg)


def parse_cli(argv: Optional[List[str]] = None, default_name: str = "config",
              default_dirs: Sequence[os.PathLike] = ()):
    """Splits a Hydra-style command line into (config_name, config_dirs, overrides)."""
    argv = list(sys.argv[1:] if argv is None else argv)
    name, dirs, overrides = default_name, [Path(d) for d in default_dirs], []
    i = 0
    while i < len(argv):
        a = argv[i]
        if a in ("--config-name", "-cn"):
            name = argv[i + 1]
            i += 2
        elif a.startswith("--config-name="):
            name = a.split("=", 1)[1]
            i += 1
        elif a in ("--config-path", "-cp", "--config-dir", "-cd"):
            dirs.insert(0, Path(argv[i + 1]))
            i += 2
        elif a.startswith(("--config-path=", "--config-dir=")):
            dirs.insert(0, Path(a.split("=", 1)[1]))
            i += 1
        else:
            overrides.append(a)
            i += 1
    if name.endswith(".yaml"):
        name = name[:-5]
    return name, dirs, overrides


def dump(cfg, path: os.PathLike):
    with open(path, "w") as f:
        yaml.safe_dump(_to_plain(cfg), f, sort_keys=False, default_flow_style=None)
