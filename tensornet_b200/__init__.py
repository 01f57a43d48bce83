"""tensornet_b200: a Blackwell-native framework for very large sparse recommendation models
with the capabilities and Python surface of Qihoo360/tensornet.

    import tensornet_b200 as tn
    tn.core.init()
"""
from . import core
from . import feature_column
from . import layers
from . import optimizer
from . import model
from . import models
from . import data
from . import metric
from . import callbacks
from . import distribute
from . import utils
from . import tools
from . import serving
from .version import VERSION as __version__

__all__ = ["core", "feature_column", "layers", "optimizer", "model", "models", "data", "metric", "callbacks",
           "distribute", "utils", "tools", "serving", "__version__"]
