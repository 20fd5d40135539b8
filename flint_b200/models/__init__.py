"""Architectures.  Importing this package registers the built-in ones."""
from . import phimoe, puledra  # noqa: F401
