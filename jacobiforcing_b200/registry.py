"""Model registry: which configuration reader and which per-rank runner serve an architecture.

`resolve(model_dir)` looks at config.json the way the engine does: "architecture" (this build's native descriptions) or
"architectures" (Hugging Face descriptions).  Runners are imported lazily so that serving one family does not load, or
build, the other's native library."""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Optional


class ModelFamily:
    def __init__(self, name: str, native_config: bool, load_config: Callable, runner: Callable):
        self.name, self.native_config, self.load_config, self.runner = name, native_config, load_config, runner


def _qwen2_config(path):
    from transformers import AutoConfig
    return AutoConfig.from_pretrained(path)


def _qwen2_runner():
    from .engine.model_runner import ModelRunner
    return ModelRunner


def _hybrid_config(path):
    from .hybrid_config import HybridConfig
    return HybridConfig.from_dir(path)


def _hybrid_runner():
    from .engine.hybrid_runner import HybridModelRunner
    return HybridModelRunner


FAMILIES: Dict[str, ModelFamily] = {
    "Qwen2ForCausalLM": ModelFamily("qwen2", False, _qwen2_config, _qwen2_runner),
    "Qwen3ForCausalLM": ModelFamily("qwen2", False, _qwen2_config, _qwen2_runner),
    "Kinetar": ModelFamily("hybrid", True, _hybrid_config, _hybrid_runner),
    "Famepel": ModelFamily("hybrid", True, _hybrid_config, _hybrid_runner),
    "Vosolorn": ModelFamily("hybrid", True, _hybrid_config, _hybrid_runner),
    "Sebavik": ModelFamily("hybrid", True, _hybrid_config, _hybrid_runner),
}


def architecture_of(model_dir: Optional[str]) -> Optional[str]:
    if model_dir is None or not os.path.isfile(os.path.join(model_dir, "config.json")):
        return None
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    if isinstance(cfg.get("architecture"), str):
        return cfg["architecture"]
    archs = cfg.get("architectures") or []
    return archs[0] if archs else None


def family_of_config(model_config) -> ModelFamily:
    """Family of an already loaded model description (native or Hugging Face)."""
    if getattr(model_config, "is_hybrid", False):
        return FAMILIES[getattr(model_config, "architecture", "Kinetar")]
    return FAMILIES["Qwen2ForCausalLM"]


def resolve(model_dir: Optional[str]) -> ModelFamily:
    arch = architecture_of(model_dir)
    if arch is None:
        return FAMILIES["Qwen2ForCausalLM"]
    if arch not in FAMILIES:
        raise NotImplementedError(f"architecture {arch!r} is not registered (known: {sorted(FAMILIES)})")
    return FAMILIES[arch]
