from .model import (Model, PCGradModel, load_done_info, save_done_info, read_last_train_dt, match_dtype_and_rank,
                    apply_mask)

__all__ = ["Model", "PCGradModel", "load_done_info", "save_done_info", "read_last_train_dt", "match_dtype_and_rank",
           "apply_mask"]
