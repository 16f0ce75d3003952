"""Architectures known to the registry.  Importing the package registers them."""

from . import llama  # noqa: F401
from .model import Model, build_model, load_model
