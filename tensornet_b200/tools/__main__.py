import argparse

from . import merge_sparse, resize_dense, resize_sparse


def main():
    ap = argparse.ArgumentParser(prog="python -m tensornet_b200.tools")
    sub = ap.add_subparsers(dest="tool", required=True)
    p = sub.add_parser("merge-sparse"); p.add_argument("table_dir"); p.add_argument("out_file"); p.add_argument("--brackets", action="store_true")
    p = sub.add_parser("resize-sparse"); p.add_argument("table_dir"); p.add_argument("out_dir"); p.add_argument("world", type=int); p.add_argument("--mode", default="txt")
    p = sub.add_parser("resize-dense"); p.add_argument("table_dir"); p.add_argument("out_dir"); p.add_argument("world", type=int); p.add_argument("--opt", default="Adam")
    a = ap.parse_args()
    if a.tool == "merge-sparse":
        print(merge_sparse(a.table_dir, a.out_file, brackets=a.brackets))
    elif a.tool == "resize-sparse":
        print(resize_sparse(a.table_dir, a.out_dir, a.world, a.mode))
    else:
        print(resize_dense(a.table_dir, a.out_dir, a.world, a.opt))


if __name__ == "__main__":
    main()
