from .features import PackedFeatures, Ragged, PACKED_KEY
from .dataset import list_files, BalanceDataset, reset_balance_dataset
from .tfrecord import TFRecordDataset, TFRecordWriter, encode_example

__all__ = ["PackedFeatures", "Ragged", "PACKED_KEY", "list_files", "BalanceDataset", "reset_balance_dataset",
           "TFRecordDataset", "TFRecordWriter", "encode_example"]
