from .features import PackedFeatures, Ragged, PACKED_KEY
from .dataset import list_files, BalanceDataset, reset_balance_dataset
from .tfrecord import TFRecordDataset, TFRecordWriter, encode_example
from .batch_cache import BatchCacheDataset, BatchCacheWriter, write_batch_cache

__all__ = ["PackedFeatures", "Ragged", "PACKED_KEY", "list_files", "BalanceDataset", "reset_balance_dataset",
           "TFRecordDataset", "TFRecordWriter", "encode_example", "BatchCacheDataset", "BatchCacheWriter", "write_batch_cache"]
