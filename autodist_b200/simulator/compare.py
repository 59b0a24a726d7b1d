"""Predicted against measured step times.

``python -m autodist_b200.simulator.compare --model bert-large --gpus 8 --single-gpu-ms 19.9 \\
      --measured AllReduce=21.62 PartitionedPS=23.54 AllReduceEF=23.79``

The measured single-GPU step already contains forward, backward and the optimizer, so the prediction for ``N`` GPUs is
that time plus the synchronisation the strategy leaves exposed. The table shows both and their ratio; with
``--fit-overlap`` the hidden fraction of the communication is re-fitted to the measurements (least squares over the
strategies given) and written back as the simulator's ``overlap``.
"""
import argparse
import json

import torch


def _capture(model_name):
    from autodist_b200 import AutoDist
    from autodist_b200.autodist import _reset_default_autodist
    from autodist_b200.resource_spec import ResourceSpec
    from autodist_b200 import strategy as S
    _reset_default_autodist()
    ad = AutoDist(resource_spec=ResourceSpec.local(num_cpus=1), strategy_builder=S.AllReduce())
    with ad.scope(), torch.device("meta" if model_name.endswith("@meta") else "cpu"):
        if model_name.startswith("bert"):
            from autodist_b200.models.bert import BertConfig, BertPretrainer, synthetic_batch
            cfg = {"bert-large": BertConfig.large, "bert-base": BertConfig.base, "bert-tiny": BertConfig.tiny}[model_name]()
            model = BertPretrainer(cfg)
            batch = synthetic_batch(cfg, 2, 32, 4)
            phs = {k: ad.placeholder((None,) + tuple(v.shape[1:]), v.dtype, name=k) for k, v in batch.items()}
            loss = model(**phs)
            opt = torch.optim.Adam(model.parameters(), lr=1e-4)
        else:
            from autodist_b200.models.cnn import ImageClassifier
            model = ImageClassifier(model_name)
            images = ad.placeholder((None, 3, 224, 224), torch.float32, name="images")
            labels = ad.placeholder((None,), torch.int64, name="labels")
            loss = model(images, labels)
            opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
        opt.minimize(loss)
        item = ad.graph_item
    _reset_default_autodist()
    return item


def builders(n):
    from autodist_b200 import strategy as S
    return {
        "AllReduce": S.AllReduce(chunk_size=256),
        "AllReduceEF": S.AllReduce(chunk_size=256, compressor="HorovodCompressorEF"),
        "Parallax": S.Parallax(chunk_size=256, reduction_devices="gpu"),
        "PSLoadBalancing": S.PSLoadBalancing(reduction_devices="gpu"),
        "PartitionedPS": S.PartitionedPS(num_shards=n, reduction_devices="gpu"),
    }


def compare(model_name, gpus, single_gpu_ms, measured, fit_overlap=False):
    from autodist_b200.resource_spec import ResourceSpec
    from autodist_b200.simulator.simulator import Simulator
    item = _capture(model_name)
    spec = ResourceSpec.local(num_gpus=gpus)
    sim = Simulator(spec)
    rows = []
    for name, b in builders(gpus).items():
        bd = sim.breakdown(b.build(item, spec), item)
        rows.append({"strategy": name, "sync_ms": bd["sync_ms"], "measured_ms": measured.get(name)})
    if fit_overlap:
        pts = [(r["sync_ms"], r["measured_ms"] - single_gpu_ms) for r in rows if r["measured_ms"]]
        den = sum(s * s for s, _ in pts)
        if den > 0:
            sim.overlap = min(1.0, max(0.0, 1.0 - sum(s * e for s, e in pts) / den))
    for r in rows:
        r["predicted_ms"] = single_gpu_ms + r["sync_ms"] * (1.0 - sim.overlap)
        r["ratio"] = r["predicted_ms"] / r["measured_ms"] if r["measured_ms"] else None
    return {"model": model_name, "gpus": gpus, "single_gpu_ms": single_gpu_ms, "overlap": sim.overlap, "rows": rows}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="bert-large")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--single-gpu-ms", type=float, required=True)
    ap.add_argument("--measured", nargs="*", default=[], help="Strategy=ms pairs")
    ap.add_argument("--fit-overlap", action="store_true")
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args()
    measured = {k: float(v) for k, v in (kv.split("=") for kv in args.measured)}
    out = compare(args.model, args.gpus, args.single_gpu_ms, measured, args.fit_overlap)
    if args.json:
        print(json.dumps(out))
        return
    print(f"{out['model']} on {out['gpus']} GPUs, single-GPU step {out['single_gpu_ms']:.2f} ms, hidden fraction {out['overlap']:.2f}")
    print(f"{'strategy':18s} {'sync ms':>9s} {'predicted':>10s} {'measured':>9s} {'pred/meas':>9s}")
    for r in out["rows"]:
        meas = f"{r['measured_ms']:9.2f}" if r["measured_ms"] else "        -"
        ratio = f"{r['ratio']:9.3f}" if r["ratio"] else "        -"
        print(f"{r['strategy']:18s} {r['sync_ms']:9.2f} {r['predicted_ms']:10.2f} {meas} {ratio}")


if __name__ == "__main__":
    main()
