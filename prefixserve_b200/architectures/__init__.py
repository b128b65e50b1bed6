"""Importing this package registers every architecture the engine ships."""

from . import llama, nerenex  # noqa: F401
