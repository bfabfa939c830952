"""Architectures.  Importing this package registers the built-in ones."""
from . import phimoe  # noqa: F401
