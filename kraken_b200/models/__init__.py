from .tp_mlp import TPMLP

__all__ = ["TPMLP"]
