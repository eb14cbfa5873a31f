"""Architectures this library can build.  Importing the package registers them."""
from . import llama, lasezen, gikepel, lomusun, tapupel  # noqa: F401
