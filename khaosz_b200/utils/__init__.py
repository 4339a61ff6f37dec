from .flat_params import FlatParameters

__all__ = ["FlatParameters"]
