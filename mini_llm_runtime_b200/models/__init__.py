"""Importing this package registers the architectures."""
from . import gopevik, qwen3  # noqa: F401
