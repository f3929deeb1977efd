"""Importing this package registers every architecture the framework ships."""
from . import gpt2  # noqa: F401
