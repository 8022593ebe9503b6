from .base import ConfigError, read_json
from .llama import LlamaConfig, RopeScaling
from .registry import (Architecture, load_config, register_architecture,
                       registered_architectures, resolve_architecture)

__all__ = ["ConfigError", "read_json", "LlamaConfig", "RopeScaling", "Architecture",
           "load_config", "register_architecture", "registered_architectures",
           "resolve_architecture"]
from .pifutar import PifutarConfig  # noqa: E402

__all__.append("PifutarConfig")
from .zupitar import ZupitarConfig  # noqa: E402

__all__.append("ZupitarConfig")
from .tizodra import TizodraConfig  # noqa: E402

__all__.append("TizodraConfig")
from .fokisun import FokisunConfig  # noqa: E402

__all__.append("FokisunConfig")
