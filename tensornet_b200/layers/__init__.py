from .embedding_features import EmbeddingFeatures
from .sequence_embedding_features import SequenceEmbeddingFeatures
from .normalization_layer import TNBatchNormalizationBase, TNBatchNormalization, PCTRDNNBatchNormalization
from .position_mapping import PositionMappingLayer
from .dense import MLP, DenseHead, FMLayer, DeepCrossLayer

__all__ = ["EmbeddingFeatures", "SequenceEmbeddingFeatures", "TNBatchNormalizationBase", "TNBatchNormalization",
           "PCTRDNNBatchNormalization", "PositionMappingLayer", "MLP", "DenseHead", "FMLayer", "DeepCrossLayer"]
