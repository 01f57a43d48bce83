"""Training driver (the role of examples/main.py in the reference): build a model under PsStrategy,
train day by day with PsWeightCheckpoint (skipping days already trained according to the
``_checkpoint`` done-file), save the dense sub-model for serving, optionally predict and dump.

    python examples/gen_example_data.py --out /tmp/tn_example_data
    python examples/main.py --data /tmp/tn_example_data --model-dir /tmp/tn_model --model wide_deep
    torchrun --nproc-per-node 2 examples/main.py ...          # one process per GPU (or CPU rank)
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

import tensornet_b200 as tn


def read_dataset(files, batch_size, slots, dense_dim, rank, world):
    """Shard files by rank, cut them into batches, balance the number of batches between ranks.  TFRecord files
    (``tf-*``, the reference's input format) go through the native reader; ``.pt`` files are sliced here."""
    mine = files[rank::world] if len(files) >= world else files
    if mine and os.path.basename(mine[0]).startswith("tf-"):
        return tn.data.BalanceDataset(tn.data.TFRecordDataset(mine, batch_size, slots, dense_keys={"dense": dense_dim} if dense_dim else None,
                                                              label_key="label", drop_remainder=True))

    def gen():
        for f in files[rank::world] if len(files) >= world else files:
            d = torch.load(f)
            n = d["label"].shape[0]
            for lo in range(0, n - batch_size + 1, batch_size):
                hi = lo + batch_size
                feats = {}
                for s in slots:
                    vals, offs = d["ids"][s]
                    o = offs[lo:hi + 1]
                    feats[s] = tn.data.Ragged(vals[o[0]:o[-1]], (o - o[0]).int())
                if dense_dim:
                    feats["dense"] = d["dense"][lo:hi]
                feats["label"] = d["label"][lo:hi]
                yield feats, d["label"][lo:hi]
    return tn.data.BalanceDataset(gen())


def list_day_files(data, days):
    """``part-*.pt`` files of the days, or their ``tf-*`` TFRecord files when there are none."""
    try:
        return tn.data.list_files(data, days, "part-*")
    except FileNotFoundError:
        return tn.data.list_files(data, days, "tf-*")


def build_model(name, slots, dense_dim, hidden, emb_dim):
    opt = tn.core.AdaGrad(learning_rate=0.01, initial_g2sum=0.1, initial_scale=0.1)
    kw = dict(dnn_hidden_units=hidden, embedding_dim=emb_dim, dense_dim=dense_dim, sparse_opt=opt, bucket_size=4096,
              target_columns=["label"])
    if name == "wide_deep":
        return tn.models.WideDeep(slots, slots, **kw)
    if name == "deepfm":
        return tn.models.DeepFM(slots, slots, **kw)
    if name == "deep_cross":
        return tn.models.DeepCross(slots, **kw)
    raise ValueError(name)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", default="/tmp/tn_example_data")
    ap.add_argument("--model-dir", default="/tmp/tn_model")
    ap.add_argument("--model", default="wide_deep", choices=["wide_deep", "deepfm", "deep_cross"])
    ap.add_argument("--days", nargs="+", default=["2020-05-10", "2020-05-11"])
    ap.add_argument("--batch-size", type=int, default=32)
    ap.add_argument("--slots", type=int, default=4)
    ap.add_argument("--dense-dim", type=int, default=0)
    ap.add_argument("--hidden", type=int, nargs="+", default=[512, 256, 256])
    ap.add_argument("--emb-dim", type=int, default=8)
    ap.add_argument("--save-mode", default="txt", choices=["txt", "bin"])
    ap.add_argument("--predict", action="store_true")
    ap.add_argument("--max-steps", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0, help="seed of the dense initialisation (the same on every rank)")
    ap.add_argument("--step-log", default="", help="append one JSON line per 100 steps (throughput, loss, table sizes) to this file")
    ap.add_argument("--profile-dir", default="", help="write a timeline of training steps 50-60 of the first day here")
    a = ap.parse_args()

    strategy = tn.distribute.PsStrategy()
    rt = tn.core.runtime()
    slots = [str(i + 1) for i in range(a.slots)]
    torch.manual_seed(a.seed)
    with strategy.scope():
        model = build_model(a.model, slots, a.dense_dim, a.hidden, a.emb_dim)
        model.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=0.001)), loss="binary_crossentropy",
                      metrics=[tn.metric.CTR(), tn.metric.PCTR(), tn.metric.COPC(), tn.metric.AUC()])

    last_dt = tn.model.read_last_train_dt(a.model_dir)
    report = {"days": []}
    for day in a.days:
        if last_dt is not None and day <= last_dt:       # already trained (resume after a restart)
            continue
        files = list_day_files(a.data, [day])
        ds = read_dataset(files, a.batch_size, slots, a.dense_dim, rt.rank, rt.world)
        cb = tn.callbacks.PsWeightCheckpoint(a.model_dir, need_save_model=True, dt=day, delta_days=1, save_mode=a.save_mode)
        t0 = time.time()
        cbs = [cb] + ([tn.utils.StepLog(a.step_log, every=100)] if a.step_log else [])
        if a.profile_dir and not report["days"]:
            cbs.append(tn.callbacks.ProfileBatches(a.profile_dir, 50, 60))
        hist = model.fit(ds, epochs=1, steps_per_epoch=a.max_steps or None, callbacks=cbs)
        steps = model.optimizer.iterations
        # the compiled metrics of the pass (fit resets them when a pass begins)
        day_metrics = {m.name.lower(): hist[m.name][-1] for m in model.metrics}
        report["days"].append({"day": day, "loss": hist["loss"][-1], "seconds": time.time() - t0, "steps": steps, **day_metrics})
        if rt.rank == 0:
            print(f"{day}: loss {hist['loss'][-1]:.5f} " + " ".join(f"{k} {v:.5f}" for k, v in day_metrics.items()), flush=True)
    if rt.rank == 0:
        os.makedirs(a.model_dir, exist_ok=True)
        torch.save(model.sub_model.state_dict(), os.path.join(a.model_dir, "sub_model.pt"))
    if a.predict:
        files = list_day_files(a.data, a.days[-1:])
        ds = read_dataset(files, a.batch_size, slots, a.dense_dim, rt.rank, rt.world)
        y, p = model.predict(ds, steps=a.max_steps or None)
        out = os.path.join(a.model_dir, "predict")
        os.makedirs(out, exist_ok=True)
        with open(os.path.join(out, "part-%05d" % rt.rank), "w") as f:
            for yy, pp in zip(y.reshape(-1).tolist(), p.reshape(-1).tolist()):
                f.write(f"{yy}\t{pp}\n")
        auc = tn.metric.AUC(); auc.update_state(y, p)
        report["predict_auc"] = auc.result()
    tn.core.barrier()
    if rt.rank == 0:
        print(json.dumps(report), flush=True)
    tn.core.shutdown()


if __name__ == "__main__":
    main()
