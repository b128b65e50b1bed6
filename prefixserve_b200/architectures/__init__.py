"""Importing this package registers every architecture the engine ships."""

from . import gekopel, llama, nerenex  # noqa: F401
