"""Architectures this package ships. Importing the package registers them."""
from . import qwen3  # noqa: F401
