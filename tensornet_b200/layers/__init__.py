from .embedding_features import EmbeddingFeatures
from .dense import MLP, DenseHead, FMLayer, DeepCrossLayer

__all__ = ["EmbeddingFeatures", "MLP", "DenseHead", "FMLayer", "DeepCrossLayer"]
