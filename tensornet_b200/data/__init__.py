from .features import PackedFeatures, Ragged, PACKED_KEY
from .dataset import list_files, BalanceDataset, reset_balance_dataset

__all__ = ["PackedFeatures", "Ragged", "PACKED_KEY", "list_files", "BalanceDataset", "reset_balance_dataset"]
