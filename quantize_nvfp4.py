"""Quantize a bf16 checkpoint directory into the NVFP4/FP8 recipe layout the engine loads.

  python quantize_nvfp4.py --model-dir IN --out OUT [--recipe all,gdn:fp8]

Writes ``stem.weight_packed`` / ``stem.weight_scale`` / ``stem.weight_global_scale`` (NVFP4),
``stem.weight`` F8_E4M3 + ``stem.weight_scale`` (FP8), copies everything else, shards at 12 GB, writes the
index, copies the tokenizer sidecars and stamps ``quantization_config`` into ``config.json``
(same as ``python -m velogb10_b200 --quantize``).
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--model-dir", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--recipe", default="all,gdn:fp8")
    ap.add_argument("--max-shard-gb", type=float, default=12.0)
    a = ap.parse_args()
    from velogb10_b200.checkpoint import io
    print(json.dumps(io.quantize_checkpoint(a.model_dir, a.out, a.recipe, int(a.max_shard_gb * (1 << 30)))))
