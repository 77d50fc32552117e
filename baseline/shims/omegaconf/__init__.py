"""Stand-in for the part of OmegaConf the reference's exec path touches (the package is not in this
image).  A DictConfig here is a dict with attribute access; interpolations are resolved by the
framework's YAML composer.  Only used by the reference arm of bench.py."""
from __future__ import annotations

import yaml

from mist_b200.utils import yamlconf


class DictConfig(yamlconf.Node):
    pass


class ListConfig(list):
    pass


def _wrap(obj):
    if isinstance(obj, dict):
        return DictConfig({k: _wrap(v) for k, v in obj.items()})
    if isinstance(obj, (list, tuple)):
        return ListConfig(_wrap(v) for v in obj)
    return obj


def _plain(obj):
    if isinstance(obj, dict):
        return {k: _plain(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_plain(v) for v in obj]
    return obj


class OmegaConf:
    @staticmethod
    def create(obj=None):
        if isinstance(obj, str):
            obj = yaml.safe_load(obj)
        return _wrap(obj if obj is not None else {})

    @staticmethod
    def resolve(cfg):
        resolved = _wrap(yamlconf.resolve(_plain(cfg)))
        cfg.clear()
        cfg.update(resolved)

    @staticmethod
    def to_container(cfg, resolve=False, **_):
        plain = _plain(cfg)
        return yamlconf.resolve(plain) if resolve else plain

    @staticmethod
    def to_yaml(cfg, resolve=False, **_):
        return yaml.safe_dump(OmegaConf.to_container(cfg, resolve=resolve), sort_keys=False)

    @staticmethod
    def load(path):
        with open(path) as f:
            return _wrap(yaml.safe_load(f) or {})

    @staticmethod
    def save(config, f, resolve=False):
        text = OmegaConf.to_yaml(config, resolve=resolve)
        if hasattr(f, "write"):
            f.write(text)
        else:
            with open(f, "w") as fh:
                fh.write(text)

    @staticmethod
    def set_struct(cfg, value):
        return None

    @staticmethod
    def is_config(obj):
        return isinstance(obj, (DictConfig, ListConfig))
