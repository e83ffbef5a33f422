"""Architectures.  Importing the package registers them by the name config.json uses."""
from . import qwen3  # noqa: F401
