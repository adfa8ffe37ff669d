"""Architectures known to the registry.  Importing the package registers them."""

from . import gavodra, lanirax, lasapel, llama, rumedra  # noqa: F401
from .model import Model, build_model, load_model
