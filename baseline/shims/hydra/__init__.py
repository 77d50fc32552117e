"""Stand-in for ``hydra.main`` (Hydra is not in this image): composes the YAML tree the decorator points
at with the framework's own composer, applies the command-line overrides and calls the function with the
result.  Only used by the reference arm of bench.py."""
from __future__ import annotations

import functools
import inspect
import os
import sys

from mist_b200.utils import yamlconf
from omegaconf import _wrap


def compose_for(func_file, config_path, config_name, argv):
    base = os.path.dirname(os.path.abspath(func_file))
    default_dir = os.path.normpath(os.path.join(base, config_path)) if config_path else base
    name, dirs, overrides = yamlconf.parse_cli(argv, default_name=config_name or "config",
                                               default_dirs=[default_dir])
    if name.endswith(".yaml"):
        name = name[:-5]
    return _wrap(yamlconf.compose(name, dirs, overrides, do_resolve=False))


def main(version_base=None, config_path=None, config_name=None):
    def deco(func):
        @functools.wraps(func)
        def wrapper(cfg=None):
            if cfg is None:
                cfg = compose_for(inspect.getsourcefile(func), config_path, config_name, sys.argv[1:])
            return func(cfg)
        return wrapper
    return deco
