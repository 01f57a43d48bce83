from .deepfm import DeepFM, DeepFMSubModel

__all__ = ["DeepFM", "DeepFMSubModel"]
