"""Architectures this package ships. Importing the package registers them."""
from . import fekulix, kovusun, mugipel, qwen3, rofozen  # noqa: F401
