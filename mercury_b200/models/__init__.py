"""Model descriptions. Importing this package registers the built-in architectures."""

from . import fegenex, kinelix, lizazen, qwen2, sisavik  # noqa: F401
from .model import Model  # noqa: F401
from .spec import LayerCall, ModelSpec  # noqa: F401
