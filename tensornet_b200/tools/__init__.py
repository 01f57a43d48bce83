"""Offline checkpoint tools (tensornet_tools/python/*.py in the reference, there as Spark jobs):

* ``merge_sparse``   - merge every block of every rank into one ``sign -> weights`` text dictionary,
                       the export used by the serving side (merge_sparse.py:34-41, utils.py:309-316)
* ``resize_sparse``  - re-shard a sparse table checkpoint to another rank count (resize_sparse.py:35-54)
* ``resize_dense``   - re-shard a dense table checkpoint (resize_dense.py:32-47)
* ``merge_extra_embedding`` - copy the embeddings of old signs onto new signs (merge_extra_embedding.py:39-83)

They run in one process on the host; command line: ``python -m tensornet_b200.tools <tool> ...``.
"""
from .ckpt_tools import merge_sparse, resize_sparse, resize_dense, merge_extra_embedding, read_sparse_table

__all__ = ["merge_sparse", "resize_sparse", "resize_dense", "merge_extra_embedding", "read_sparse_table"]
