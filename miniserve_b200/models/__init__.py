"""Architectures this package ships. Importing the package registers them."""
from . import fekulix, mugipel, qwen3, rofozen  # noqa: F401
