"""Shared command-line plumbing of the three entry points."""
from __future__ import annotations

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from mist_b200.config import CONFIG_DIR, MistConfig  # noqa: E402
from mist_b200.utils import yamlconf  # noqa: E402


def load_from_cli(argv=None, check_world_size=True):
    """Hydra-style command line -> (MistConfig, raw node).  Extra config directories:
    ``benchmark/mist_b200/configs`` (user files) then the packaged tree."""
    name, dirs, overrides = yamlconf.parse_cli(argv, default_name="config")
    search = list(dirs) + [os.path.join(HERE, "configs"), CONFIG_DIR]
    search = [d for d in search if os.path.isdir(d)]
    node = yamlconf.compose(name, search, overrides)
    return MistConfig.from_dict_config(node, check_world_size=check_world_size), node


def output_dir(node) -> str:
    out = node.get("output_dir") or os.getcwd()
    os.makedirs(out, exist_ok=True)
    return out
