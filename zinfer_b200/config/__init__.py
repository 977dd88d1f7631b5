from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule
from .qwen3 import ConfigError, Qwen3Config, qwen3_model_spec
from .registry import (Family, UnknownArchitecture, family_for, load_config, register_family, registered,
                       unregister_family)

register_family(Family(name="Qwen3ForCausalLM", model_type="qwen3", config_class=Qwen3Config,
                       model_spec=qwen3_model_spec), replace=True)

__all__ = [
    "ConfigError", "Family", "LayerSpec", "ModelSpec", "PartSpec", "Qwen3Config", "ScheduleEntry",
    "UnknownArchitecture", "default_schedule", "family_for", "load_config", "qwen3_model_spec",
    "register_family", "registered", "unregister_family",
]
