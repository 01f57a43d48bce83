from .deepfm import DeepFM, DeepFMSubModel
from .wide_deep import WideDeep, WideDeepSubModel
from .deep_cross import DeepCross, DCNv2, CrossV2, DeepCrossSubModel, DCNv2SubModel

__all__ = ["DeepFM", "DeepFMSubModel", "WideDeep", "WideDeepSubModel", "DeepCross", "DCNv2", "CrossV2",
           "DeepCrossSubModel", "DCNv2SubModel"]
