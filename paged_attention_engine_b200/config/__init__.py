from .model_spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .engine_config import EngineConfig
from .errors import ConfigError
from .bidonex import BidonexConfig
from .finezen import FinezenConfig
from .qwen2 import Qwen2Config
from .pukerax import PukeraxConfig
from .zugarax import ZugaraxConfig
from .registry import ARCHITECTURES, Architecture, register_architecture, resolve, resolve_folder

__all__ = [
    "ARCHITECTURES", "Architecture", "BidonexConfig", "ConfigError", "EngineConfig", "FinezenConfig", "LayerSpec", "ModelSpec", "PartSpec", "Qwen2Config",
    "PukeraxConfig", "ScheduleEntry", "ZugaraxConfig", "register_architecture", "resolve", "resolve_folder",
]
