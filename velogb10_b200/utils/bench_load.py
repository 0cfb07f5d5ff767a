"""Checkpoint load from disk, timed: writes a synthetic quantised checkpoint of the chosen shape (the recipe layout the
offline quantiser produces), drops nothing from the page cache (no privileges needed), then builds the model from the
directory twice: through the read-ahead workers and through the plain lazy reader. Prints one JSON line per arm with
the byte count, wall time, effective GB/s and the read / wait / build split of the ``[load]`` line.

  python -m velogb10_b200.utils.bench_load --model 27b --layers 16 --dir /tmp/velo_ckpt

The files were just written, so reads are served from the page cache: the figure is the loader's own overhead
(parse, pinned memcpy, upload, GPU tiling), the ceiling a real disk would sit under.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import time

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="27b")
    ap.add_argument("--layers", type=int, default=16, help="keep only the first N layers (0 = full depth)")
    ap.add_argument("--dir", default="/tmp/velo_ckpt")
    ap.add_argument("--recipe", default="all")
    ap.add_argument("--workers", default="4,0")
    ap.add_argument("--keep", action="store_true")
    args = ap.parse_args()

    from ..checkpoint import io
    from ..checkpoint.synthetic import SyntheticSource
    from ..config import ModelConfig, preset
    from ..models.weights import ModelBuilder

    dev = "cuda" if torch.cuda.is_available() else "cpu"
    cfg = preset(args.model, mtp=True)
    if args.layers and args.layers < cfg.num_layers:
        cfg.num_layers = args.layers
        cfg.layer_types = cfg.layer_types[:args.layers]
    if os.path.exists(args.dir):
        shutil.rmtree(args.dir)
    syn = SyntheticSource(cfg, 0, dev)
    t0 = time.time()
    stats = io.write_checkpoint(args.dir, ((n, syn.get(n)) for n in syn.names()), cfg.to_hf_dict(), args.recipe,
                                max_shard_bytes=4 << 30)
    print(json.dumps({"wrote": args.dir, "gb": round(stats["bytes"] / 1e9, 3), "seconds": round(time.time() - t0, 1),
                      "tensors": {k: stats[k] for k in ("nvfp4", "fp8", "copied")}}), flush=True)
    cfg2 = ModelConfig.from_json(os.path.join(args.dir, "config.json"))
    for w in [int(x) for x in args.workers.split(",")]:
        if dev == "cuda":
            torch.cuda.synchronize()
        t0 = time.time()
        src = io.open_checkpoint(args.dir, dev, workers=w)
        model = ModelBuilder(cfg2, src, recipe="off", device=dev).build()
        if dev == "cuda":
            torch.cuda.synchronize()
        dt = time.time() - t0
        row = {"arm": f"read-ahead x{w}" if w else "plain lazy reader", "seconds": round(dt, 2),
               "gb_per_s": round(stats["bytes"] / 1e9 / dt, 2), "report": io.load_report(src, dt)}
        if hasattr(src, "close"):
            src.close()
        print(json.dumps(row), flush=True)
        del model
        if dev == "cuda":
            torch.cuda.empty_cache()
    if not args.keep:
        shutil.rmtree(args.dir)


if __name__ == "__main__":
    main()
