VERSION = "0.1.0"
#: version of the reference whose API surface and checkpoint formats are reproduced
REFERENCE_VERSION = "0.208.0.post1"
