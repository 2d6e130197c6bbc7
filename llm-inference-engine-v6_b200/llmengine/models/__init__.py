"""Architectures: each module registers one name of config.json `architectures`."""
from . import llama  # noqa: F401
