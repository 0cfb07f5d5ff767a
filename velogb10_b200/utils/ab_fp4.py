"""A/B of the two decode-width GEMM numerics on one model: the block-scaled FP4 tensor-core path (weights consumed
packed, each activation row expanded to a four-term NVFP4 series) against the 16-bit path (weights dequantised to
f16 exactly, f16 activations), same weights, same tokens. Reports, per decode step, the relative L2 difference of the
full-vocabulary logits, the greedy-token agreement over a free-running generation, and the negative log-likelihood
each path assigns to the other's tokens (a perplexity-style score on the same text).

  python -m velogb10_b200.utils.ab_fp4 --model 27b --layers 16 --prompt 512 --new 256
"""
from __future__ import annotations

import argparse
import json

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="27b")
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--std", type=float, default=0.02)
    args = ap.parse_args()
    from ..checkpoint.synthetic import SyntheticSource
    from ..config import preset
    from ..models.runtime import GpuModel
    from ..models.weights import ModelBuilder
    from ..ops import lib as vlib
    dev = "cuda"
    cfg = preset(args.model, mtp=False)
    if args.layers and args.layers < cfg.num_layers:
        cfg.num_layers = args.layers
        cfg.layer_types = cfg.layer_types[:args.layers]
    w = ModelBuilder(cfg, SyntheticSource(cfg, 0, dev, args.std), recipe="all", device=dev).build()
    gm = GpuModel(w, device=dev)
    gm.alloc_state(2, 2 + 17, args.prompt + args.new + 8)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (args.prompt,), generator=g).tolist()

    def run(fp4: bool, slot: int, forced=None):
        gm.use_fp4 = fp4
        gm.zero_slot(slot)
        lg, _ = gm.prefill(slot, prompt, 0, want_hidden=False)
        toks, logits = [], []
        tok = int(lg.argmax()) if forced is None else forced[0]
        for i in range(args.new):
            toks.append(tok)
            lgd, _ = gm.decode([tok], [args.prompt + i], [slot])
            logits.append(lgd[0].float().clone())
            tok = int(lgd[0].argmax()) if forced is None else (forced[i + 1] if i + 1 < len(forced) else 0)
        return toks, logits

    # free-running generations (token agreement), then the 16-bit path re-run on the FP4 path's tokens so the logits
    # of both paths can be compared position by position on identical inputs
    t4, l4 = run(True, 0)
    t16, _ = run(False, 1)
    agree = 0
    while agree < args.new and t4[agree] == t16[agree]:
        agree += 1
    _, l16f = run(False, 1, forced=t4 + [0])
    vlib.check_err_word()
    rel = [((a - b).norm() / b.norm()).item() for a, b in zip(l4, l16f)]
    top1 = sum(int(a.argmax()) == int(b.argmax()) for a, b in zip(l4, l16f)) / len(l4)
    nxt = torch.tensor(t4[1:], device=dev)
    nll = lambda L: float(torch.stack([-torch.log_softmax(x, -1)[t] for x, t in zip(L[:-1], nxt)]).mean())
    print(json.dumps({"model": cfg.name, "layers": cfg.num_layers, "prompt": args.prompt, "new_tokens": args.new,
                      "logits_rel_l2": {"first": rel[0], "median": sorted(rel)[len(rel) // 2], "max": max(rel), "last": rel[-1]},
                      "same_argmax_on_identical_inputs": top1, "free_running_tokens_equal_until": agree,
                      "free_running_agreement": sum(a == b for a, b in zip(t4, t16)) / args.new,
                      "nll_of_fp4_path_tokens": {"fp4_path": nll(l4), "f16_path": nll(l16f)},
                      "ppl": {"fp4_path": float(torch.tensor(nll(l4)).exp()), "f16_path": float(torch.tensor(nll(l16f)).exp())}}))


if __name__ == "__main__":
    main()
