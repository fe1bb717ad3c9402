"""Architectures.  Importing this package registers them."""
from . import bedenex, llama, redarax, vufolorn  # noqa: F401
