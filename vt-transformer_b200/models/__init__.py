"""Models.  Importing the package registers the built-in architectures."""
from . import qwen2  # noqa: F401
from .base import DecoderModel
