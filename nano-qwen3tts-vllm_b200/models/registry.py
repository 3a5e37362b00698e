"""Architecture registry: ``config.json`` -> configuration class, model class, runner and engine.

A checkpoint names its design in ``"architecture"``; Qwen3-TTS checkpoints (which predate the key) are recognised by
their ``talker_config``.  Entries hold import paths, so looking one up imports nothing it does not need."""
from __future__ import annotations

import importlib
from dataclasses import dataclass


@dataclass(frozen=True)
class Architecture:
    name: str
    config: str            # "module:Class" relative to the package
    model: str
    runner: str
    engine: str

    def _get(self, path: str):
        mod, cls = path.split(":")
        return getattr(importlib.import_module(mod, __package__.rsplit(".", 1)[0]), cls)

    @property
    def config_cls(self):
        return self._get(self.config)

    @property
    def model_cls(self):
        return self._get(self.model)

    @property
    def runner_cls(self):
        return self._get(self.runner)

    @property
    def engine_cls(self):
        return self._get(self.engine)


ARCHITECTURES: dict[str, Architecture] = {}


def register(arch: Architecture) -> None:
    ARCHITECTURES[arch.name] = arch


register(Architecture("Qwen3TTS", ".config:ModelConfig", ".models.qwen3_tts_talker:Qwen3TTSTalkerForCausalLM",
                      ".engine.model_runner.talker_mode_runner:TalkerModeModelRunner",
                      ".engine.llm_engine.talker_llm_engine:TalkerLLMEngine"))
register(Architecture("Bokenex", ".config:BokenexConfig", ".models.bokenex:BokenexForCausalLM",
                      ".engine.model_runner.lm_model_runner:LMModelRunner",
                      ".engine.llm_engine.lm_engine:CausalLMEngine"))


register(Architecture("Ridevik", ".config:RidevikConfig", ".models.ridevik:RidevikForCausalLM",
                      ".engine.model_runner.lm_model_runner:LMModelRunner",
                      ".engine.llm_engine.lm_engine:CausalLMEngine"))
register(Architecture("Tibivik", ".config:TibivikConfig", ".models.tibivik:TibivikForCausalLM",
                      ".engine.model_runner.lm_model_runner:LMModelRunner",
                      ".engine.llm_engine.lm_engine:CausalLMEngine"))
register(Architecture("Teberax", ".config:TeberaxConfig", ".models.teberax:TeberaxForCausalLM",
                      ".engine.model_runner.lm_model_runner:LMModelRunner",
                      ".engine.llm_engine.lm_engine:CausalLMEngine"))


def resolve(config: dict) -> Architecture:
    name = config.get("architecture")
    if name is None and "talker_config" in config:
        name = "Qwen3TTS"
    if name not in ARCHITECTURES:
        raise ValueError(f"no model registered for architecture {name!r} (known: {sorted(ARCHITECTURES)})")
    return ARCHITECTURES[name]


def resolve_config_object(cfg) -> Architecture:
    """The entry whose configuration class ``cfg`` is an instance of."""
    for arch in ARCHITECTURES.values():
        if type(cfg).__name__ == arch.config.split(":")[1]:
            return arch
    raise ValueError(f"no model registered for configuration {type(cfg).__name__}")
