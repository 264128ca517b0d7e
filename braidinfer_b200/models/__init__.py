"""Architectures: how a configuration becomes a description of parts, and the
registry from config.json's architecture name to that recipe."""
from .registry import ARCHITECTURES, Architecture, architecture_for, complete_config, register_architecture
from . import bidinex, birepel, loduzen, ludazen, mistral  # noqa: F401  (registration)
from .decoder import DecoderModel
