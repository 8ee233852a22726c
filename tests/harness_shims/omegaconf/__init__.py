"""Minimal stand-in for the parts of ``omegaconf`` the reference's tools/profile_*.py use (DictConfig with attribute
access and ``.get``, ``OmegaConf.to_container / to_yaml / create``).  Test infrastructure: put on ``sys.path`` only
when the real package is not installed, so that the reference's harnesses can be imported and run unchanged."""
import yaml


class DictConfig(dict):
    def __init__(self, data=None):
        super().__init__()
        for k, v in (data or {}).items():
            self[k] = _wrap(v)

    def __getattr__(self, name):
        try:
            return self[name]
        except KeyError:
            raise AttributeError(name) from None

    def __setattr__(self, name, value):
        self[name] = _wrap(value)


class ListConfig(list):
    def __init__(self, data=()):
        super().__init__(_wrap(v) for v in data)


def _wrap(v):
    if isinstance(v, (DictConfig, ListConfig)):
        return v
    if isinstance(v, dict):
        return DictConfig(v)
    if isinstance(v, (list, tuple)):
        return ListConfig(v)
    return v


def _plain(v):
    if isinstance(v, dict):
        return {k: _plain(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [_plain(x) for x in v]
    return v


class OmegaConf:
    @staticmethod
    def create(obj=None):
        return _wrap(obj if obj is not None else {})

    @staticmethod
    def to_container(cfg, resolve=True, **_):
        return _plain(cfg)

    @staticmethod
    def to_yaml(cfg, **_):
        return yaml.safe_dump(_plain(cfg), sort_keys=False)

    @staticmethod
    def load(path):
        with open(path) as fh:
            return _wrap(yaml.safe_load(fh))
