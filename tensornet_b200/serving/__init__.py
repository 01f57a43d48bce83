"""Serving path: export the sparse dictionary, load it into a read-only GPU hash table and run the
dense sub-model on looked-up embeddings inside one CUDA graph.

In the reference, inference needs "the exported sparse dictionary plus the ordinary dense
sub-graph" (README.md:42-44): the dictionary is ``sign -> w[0..dim)`` cut out of the sparse blocks
(tensornet_tools/python/merge_sparse.py:34-41) and the dense sub-model is compiled ahead of time
(doc/tutorial/04-deploy-tf-graph-online.ipynb); its online demo fakes the lookup
(examples/online_serving/main.cc:76-81).  Here the lookup is real.
"""
from .engine import EmbeddingDictionary, InferenceEngine, ShardedInferenceEngine, export_sparse_dictionary
from .export import export_tower

__all__ = ["EmbeddingDictionary", "InferenceEngine", "ShardedInferenceEngine", "export_sparse_dictionary", "export_tower"]
