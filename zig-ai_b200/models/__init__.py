"""Architectures: each module registers its name, its config class and the function that lays out
its layers from parts."""
from . import lfm2  # noqa: F401  (registration)
from .model import Model
from ..config.base import lookup_architecture


def build_model(cfg) -> Model:
    """The model that the configuration's architecture name stands for."""
    _, build_spec = lookup_architecture(cfg.architecture)
    return Model(build_spec(cfg))
