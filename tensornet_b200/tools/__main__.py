import argparse

from . import merge_sparse, resize_dense, resize_sparse


def main():
    ap = argparse.ArgumentParser(prog="python -m tensornet_b200.tools")
    sub = ap.add_subparsers(dest="tool", required=True)
    p = sub.add_parser("merge-sparse"); p.add_argument("table_dir"); p.add_argument("out_file"); p.add_argument("--brackets", action="store_true")
    p = sub.add_parser("resize-sparse"); p.add_argument("table_dir"); p.add_argument("out_dir"); p.add_argument("world", type=int); p.add_argument("--mode", default="txt")
    p = sub.add_parser("resize-dense"); p.add_argument("table_dir"); p.add_argument("out_dir"); p.add_argument("world", type=int); p.add_argument("--opt", default="Adam")
    p = sub.add_parser("batch-cache", help="parse TFRecord files once and store the pass as ready-made batches")
    p.add_argument("out_file"); p.add_argument("files", nargs="+"); p.add_argument("--batch-size", type=int, required=True)
    p.add_argument("--slots", nargs="+", required=True); p.add_argument("--dense", nargs=2, metavar=("NAME", "WIDTH"))
    p.add_argument("--label", default="label"); p.add_argument("--single-hot", action="store_true")
    p.add_argument("--default-id", type=int, default=0); p.add_argument("--workers", type=int, default=4)
    a = ap.parse_args()
    if a.tool == "batch-cache":
        from ..data import TFRecordDataset, write_batch_cache
        ds = TFRecordDataset(a.files, a.batch_size, a.slots, dense_keys={a.dense[0]: int(a.dense[1])} if a.dense else None,
                             label_key=a.label, packed=True, single_hot=a.single_hot, default_id=a.default_id,
                             num_workers=a.workers, pin_memory=False)
        print(write_batch_cache(a.out_file, ds, a.slots, dense_name="dense" if a.dense else None, label=bool(a.label)))
    elif a.tool == "merge-sparse":
        print(merge_sparse(a.table_dir, a.out_file, brackets=a.brackets))
    elif a.tool == "resize-sparse":
        print(resize_sparse(a.table_dir, a.out_dir, a.world, a.mode))
    else:
        print(resize_dense(a.table_dir, a.out_dir, a.world, a.opt))


if __name__ == "__main__":
    main()
