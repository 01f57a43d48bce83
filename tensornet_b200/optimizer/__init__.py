from .optimizer import Optimizer, PCGrad

__all__ = ["Optimizer", "PCGrad"]
