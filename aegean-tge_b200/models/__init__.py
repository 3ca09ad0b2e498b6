"""Model assembly.  Importing this package registers the architectures it holds."""
from . import kokolorn, lepizen, mozepel, puputar, qwen2  # noqa: F401  (registration)
from .decoder import DecoderModel

__all__ = ["DecoderModel"]
