"""Model registry: which loader serves a checkpoint folder, chosen by its config.json.

A language-model checkpoint names its design in `architecture` (or, in the Hugging Face layout, in `architectures` / `model_type`).
`load_model(path)` reads config.json, looks the design up and returns what the design's loader builds: a step engine
(leopard_b200/seqlm.py) for the decoder-only language models, the plugin classes for the Leopard vision-language models."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Callable, Dict

_LOADERS: Dict[str, Callable] = {}


def register(architecture: str, loader: Callable) -> None:
    _LOADERS[architecture] = loader


def architectures():
    return sorted(_LOADERS)


def architecture_of(config: dict) -> str:
    if "architecture" in config:
        return str(config["architecture"])
    archs = config.get("architectures") or []
    if archs:
        return str(archs[0])
    return str(config.get("model_type", ""))


def load_model(path, **kw):
    path = Path(path)
    cfg_file = path / "config.json"
    if not cfg_file.exists():
        raise FileNotFoundError(f"{cfg_file} not found")
    arch = architecture_of(json.loads(cfg_file.read_text()))
    if arch not in _LOADERS:
        raise KeyError(f"no loader for architecture {arch!r}; known: {', '.join(architectures())}")
    return _LOADERS[arch](path, **kw)


def _zudalorn(path, **kw):
    from . import zudalorn
    return zudalorn.load(path, **kw)


def _ronelorn(path, **kw):
    from . import ronelorn
    return ronelorn.load(path, **kw)


def _gavatar(path, **kw):
    from . import gavatar
    return gavatar.load(path, **kw)


def _kamosun(path, **kw):
    from . import kamosun
    return kamosun.load(path, **kw)


def _llava(path, **kw):
    from .hf import myLlavaForConditionalGeneration
    return myLlavaForConditionalGeneration.from_pretrained(path, **kw)


register("Zudalorn", _zudalorn)
register("Ronelorn", _ronelorn)
register("Gavatar", _gavatar)
register("Kamosun", _kamosun)
register("LlavaForConditionalGeneration", _llava)
register("myLlavaForConditionalGeneration", _llava)
register("llava", _llava)
