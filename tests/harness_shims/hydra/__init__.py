"""Minimal stand-in for ``hydra.main`` as the reference's tools/profile_*.py use it: read
``<script dir>/<config_path>/<config_name>.yaml`` with PyYAML, apply ``key=value`` overrides from the command
line (dotted keys, YAML-parsed values), and call the decorated function with the result.  Test infrastructure:
put on ``sys.path`` only when the real package is not installed."""
import functools
import os
import sys

import yaml
from omegaconf import OmegaConf


def _apply(cfg, key, value):
    node = cfg
    parts = key.lstrip("+").split(".")
    for part in parts[:-1]:
        node = node.setdefault(part, {})
    node[parts[-1]] = yaml.safe_load(value)


def main(version_base=None, config_path=None, config_name=None):
    def decorate(fn):
        @functools.wraps(fn)
        def run(cfg=None, overrides=None):
            if cfg is None:
                base = os.path.dirname(os.path.abspath(sys.modules[fn.__module__].__file__))
                with open(os.path.join(base, config_path or "", f"{config_name}.yaml")) as fh:
                    data = yaml.safe_load(fh) or {}
                for item in (sys.argv[1:] if overrides is None else overrides):
                    if "=" in item:
                        _apply(data, *item.split("=", 1))
                cfg = OmegaConf.create(data)
            return fn(cfg)
        return run
    return decorate
