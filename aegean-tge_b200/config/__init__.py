"""Typed configurations and the architecture-independent model description."""
from .model_spec import LayerSpec, ModelSpec, PartSpec, expected_tensors
from .qwen2 import ARCHITECTURE as QWEN2_ARCHITECTURE
from .common import ConfigError, read_config_json
from .qwen2 import Qwen2Config
from .lepizen import ARCHITECTURE as LEPIZEN_ARCHITECTURE
from .lepizen import LepizenConfig
from .mozepel import ARCHITECTURE as MOZEPEL_ARCHITECTURE
from .mozepel import MozepelConfig
from .puputar import ARCHITECTURE as PUPUTAR_ARCHITECTURE
from .puputar import PuputarConfig
from .kokolorn import ARCHITECTURE as KOKOLORN_ARCHITECTURE
from .kokolorn import KokolornConfig

__all__ = ["KokolornConfig", "KOKOLORN_ARCHITECTURE", "PuputarConfig", "PUPUTAR_ARCHITECTURE", "LayerSpec", "ModelSpec", "PartSpec", "expected_tensors", "ConfigError",
           "Qwen2Config", "QWEN2_ARCHITECTURE", "LepizenConfig", "LEPIZEN_ARCHITECTURE", "MozepelConfig", "MOZEPEL_ARCHITECTURE",
           "read_config_json"]
