"""Architectures this engine builds.  Importing a module registers its architecture name."""
from . import bilolorn, desilorn, kusolorn, qwen3, zinunex  # noqa: F401
