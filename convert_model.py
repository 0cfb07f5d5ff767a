"""Convert a Hugging Face checkpoint directory into the engine's bf16 layout: per-expert MoE tensors are
fused into stacked ``experts.gate_up_proj`` / ``experts.down_proj``, everything else is copied, shards
are rewritten with an index and the tokenizer sidecars travel along. With ``--synthetic NAME`` it writes a
seeded random-init checkpoint of a preset shape instead (no download needed).

  python convert_model.py --model-dir HF_DIR --out OUT
  python convert_model.py --synthetic tiny --out OUT [--recipe off|all|all,gdn:fp8]
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--model-dir")
    ap.add_argument("--synthetic")
    ap.add_argument("--out", required=True)
    ap.add_argument("--recipe", default="off")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    from velogb10_b200.checkpoint import io
    if a.synthetic:
        from velogb10_b200.checkpoint.synthetic import synthetic_state_dict
        from velogb10_b200.config import preset
        from velogb10_b200.server.tokenizer import DEFAULT_TEMPLATE, build_byte_tokenizer
        cfg = preset(a.synthetic)
        stats = io.write_checkpoint(a.out, synthetic_state_dict(cfg, a.seed).items(), cfg.to_hf_dict(), a.recipe)
        build_byte_tokenizer().save(os.path.join(a.out, "tokenizer.json"))
        with open(os.path.join(a.out, "chat_template.jinja"), "w") as f:
            f.write(DEFAULT_TEMPLATE)
    else:
        src = io.SafetensorsSource(a.model_dir)
        with open(os.path.join(a.model_dir, "config.json")) as f:
            config = json.load(f)
        stats = io.write_checkpoint(a.out, ((n, src.get(n)) for n in src.names()), config, a.recipe,
                                    sidecar_dir=a.model_dir)
    print(json.dumps(stats))
