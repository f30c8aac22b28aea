"""Architectures.  Importing this package registers each of them."""
from . import lenuzen, nevurax, qwen2, redirax, rufisun  # noqa: F401
from .lenuzen import LenuzenConfig
from .nevurax import NevuraxConfig
from .qwen2 import Qwen2Config
from .redirax import RediraxConfig
from .rufisun import RufisunConfig

__all__ = ["LenuzenConfig", "NevuraxConfig", "Qwen2Config", "RediraxConfig", "RufisunConfig"]
