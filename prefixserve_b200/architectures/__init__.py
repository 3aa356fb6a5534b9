"""Importing this package registers every architecture the engine ships."""

from . import gekopel, goganex, llama, nerenex, zomolix  # noqa: F401
