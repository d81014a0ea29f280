"""Imports every model module so their @register_model decorators run."""
from . import llama  # noqa: F401
