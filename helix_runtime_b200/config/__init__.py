from .errors import ConfigError
from .llama import LlamaConfig
from .medolorn import MedolornConfig
from .rekasun import RekasunConfig
from .rorovik import RorovikConfig
from .zuzadra import ZuzadraConfig
from .registry import (Architecture, architecture_for, known_architectures, load_config,
                       read_config_json, register_architecture)
from .spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry

__all__ = [
    "Architecture", "BlockSpec", "ConfigError", "LlamaConfig", "MedolornConfig", "ModelSpec", "PartSpec", "RekasunConfig", "RorovikConfig",
    "ZuzadraConfig",
    "ScheduleEntry", "architecture_for", "known_architectures", "load_config",
    "read_config_json", "register_architecture",
]
