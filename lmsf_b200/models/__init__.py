"""Architectures.  Importing this package registers them."""
from . import bedenex, llama, redarax, vufolorn, zonidra  # noqa: F401
