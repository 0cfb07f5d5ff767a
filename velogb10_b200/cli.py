"""Command line: ``python -m velogb10_b200 <mode> [--flag value | --flag=value] ...``

Modes and flags keep the reference's semantics (reference: src/main.rs:5-214, :216-442, :450-494,
:2403-2890): ``--server`` (OpenAI API), ``--quantize`` / ``--requant-gdn`` (offline recipe tools),
``--generate`` (one-shot greedy), and the probe / bench / gate modes implemented in
``velogb10_b200.gates``. ``--tp N`` is a tensor-parallel degree over the GPUs of this box: launch N
processes with ``torchrun`` (one per GPU) and every rank serves in lockstep, rank 0 owning the HTTP port.
Flags are also bridged to environment variables (``VELO_*``) that deep code reads.
"""
from __future__ import annotations

import json
import os
import sys
import time
from typing import Dict, List, Optional

FLAG_ENV = {
    "--kv-cache": "VELO_KV_QUANT", "--no-decode-graphs": "VELO_NO_DECODE_GRAPHS",
    "--cpu-sample": "VELO_CPU_SAMPLE",           # engine/scheduler.py: token selection on the host from copied logits
    "--prefill-scalar": "VELO_PREFILL_SCALAR",   # models/runtime.py: exact per-token prefill kernels (no tensor-core
                                                 # attention, no chunked GatedDeltaNet); bit-identical to stepping
    "--zero-kv": "VELO_ZERO_KV", "--draft-vocab": "VELO_DRAFT_VOCAB",
    "--tp-trace": "VELO_TP_TRACE",               # engine/scheduler.py: step-latency percentiles on stderr
    "--tp-nccl": "VELO_TP_NCCL",
}
# Flags of the reference's command line that select between code paths this engine has only one of. They are
# accepted so existing launch scripts keep working, and each use is reported on stderr with the reason.
NO_EFFECT = {
    "--fuse-residual": "the residual add is always fused into the RMSNorm kernel",
    "--tp-fp32-partials": "tensor-parallel partial sums are always exchanged and added in fp32",
    "--no-shard-mixers": "attention and GatedDeltaNet mixers are always head-sharded under --tp",
    "--no-gqpack": "decode attention always serves a KV head's whole query group from one pass over its keys",
}
BOOL_FLAGS = {"--server", "--quantize", "--requant-gdn", "--generate", "--help", "-h", "--no-decode-graphs",
              "--fuse-residual", "--cpu-sample", "--prefill-scalar", "--zero-kv", "--tp-trace", "--tp-fp32-partials",
              "--no-shard-mixers", "--tp-nccl", "--no-gqpack", "--probe-binv", "--bench-verify", "--bench-mtp",
              "--bench-mtp-sample", "--bench-tree", "--bench-lanes", "--bench-prefill", "--bench-batch", "--probe-state",
              "--probe-reject", "--probe-bandwidth", "--probe-bandwidth-sustained", "--probe-gemm", "--sweep-gemm",
              "--probe-moe", "--capture-layers", "--dump-argmax", "--profile-mtp", "--perplexity", "--tp-barrier-bench",
              "--net-test", "--probe-tp-gemv", "--bench-accept", "--cpu"}

HELP = """velogb10_b200 - Blackwell-native inference engine for hybrid GatedDeltaNet + GQA models

modes
  --server                serve the OpenAI-compatible API
  --generate              one-shot greedy generation (--prompt TEXT | --prompt-ids 1,2,3) --max-new N
  --quantize              --model-dir IN --out DIR [--recipe all,gdn:fp8]   write the NVFP4/FP8 recipe layout
  --requant-gdn           --from MIXED_DIR --out DIR                       derive a gdn4 checkpoint
  gates / probes          --probe-binv --bench-verify [--draws N --seed S] --probe-state --probe-reject
                          --bench-mtp --bench-mtp-sample --bench-tree --bench-lanes --bench-accept
                          --bench-prefill --bench-batch --profile-mtp --perplexity --probe-bandwidth[-sustained]
                          --probe-gemm --sweep-gemm --probe-tp-gemv --probe-moe --capture-layers --dump-argmax
                          --tp-barrier-bench --net-test

model selection
  --model-dir DIR         checkpoint directory (config.json, safetensors, tokenizer files)
  --synthetic NAME        seeded random-init model: tiny | tiny-moe | tiny-hy3 | 27b | 35b-a3b | 122b-a10b
  --recipe SPEC           load-time quantization for bf16 checkpoints / synthetic models (default all)
  --model-name NAME       id reported by /v1/models (default: derived from the directory)
  --tokenizer PATH        tokenizer.json (default: MODEL_DIR/tokenizer.json)

server
  --port 8000  --max-batch 8  --max-tokens 8192  --max-seq-len 4096
  --mtp auto|on|off  --mtp-depth N  --ngram-draft N  --tree-draft on|off  --mtp-lanes on|off
  --prefix-cache on|off  --default-{repetition,presence,frequency}-penalty X  --reasoning-effort E
  --kv-cache bf16|q4  --no-decode-graphs  --zero-kv  --cpu-sample  --draft-vocab N
  --tp N                  tensor-parallel degree (run under torchrun with N processes)
  --tp-nccl               use library collectives instead of the fused peer-memory kernels (baseline)
  --cpu                   run the fp32 CPU oracle instead of the CUDA runtime (tiny models, tests)
"""


def parse_args(argv: List[str]) -> Dict[str, str]:
    """``--k v`` or ``--k=v``; boolean flags take no value."""
    out: Dict[str, str] = {}
    i = 0
    while i < len(argv):
        a = argv[i]
        if not a.startswith("-"):
            raise SystemExit(f"unexpected argument {a!r}")
        if "=" in a:
            k, v = a.split("=", 1)
            out[k] = v
        elif a in BOOL_FLAGS or i + 1 >= len(argv) or argv[i + 1].startswith("--"):
            out[a] = "1"
        else:
            out[a] = argv[i + 1]
            i += 1
        i += 1
    return out


def env_bridge(args: Dict[str, str]):
    for flag, env in FLAG_ENV.items():
        if flag in args:
            os.environ[env] = args[flag]
    for flag, why in NO_EFFECT.items():
        if flag in args:
            print(f"[cli] {flag} has no effect: {why}", file=sys.stderr)


def on(v: Optional[str], default: bool) -> bool:
    return default if v is None else v.lower() in ("1", "on", "true", "yes")


def derive_model_name(args: Dict[str, str]) -> str:
    if "--model-name" in args:
        return args["--model-name"]
    if "--model" in args:
        return args["--model"]
    if "--model-dir" in args:
        return os.path.basename(os.path.normpath(args["--model-dir"])) or "model"
    return args.get("--synthetic", "model")


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def load_runner(args: Dict[str, str], max_batch: int, max_seq: int):
    """Build the model runner (CUDA runtime, or the CPU oracle with --cpu) and its tokenizer."""
    import torch
    from .config import ModelConfig, preset
    from .models.weights import ModelBuilder
    from .server.tokenizer import ChatTokenizer, DEFAULT_TEMPLATE, build_byte_tokenizer
    rank, world, local = dist_env()
    tp = int(args.get("--tp", world))
    cpu = "--cpu" in args
    device = "cpu" if cpu else f"cuda:{local}"
    comm = None
    if tp > 1:
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group("gloo" if cpu else "nccl")
        if not cpu:
            torch.cuda.set_device(local)
            from .parallel.comm import TpComm
            comm = TpComm(rank, tp, torch.device(device), use_nccl="--tp-nccl" in args)
    if "--model-dir" in args:
        from .checkpoint.io import open_checkpoint
        d = args["--model-dir"]
        cfg = ModelConfig.from_json(os.path.join(d, "config.json"))
        src = open_checkpoint(d, device)
        recipe = args.get("--recipe", "off")
        tok = ChatTokenizer.from_dir(d, args.get("--tokenizer"))
    else:
        from .checkpoint.synthetic import SyntheticSource
        cfg = preset(args.get("--synthetic", "tiny"))
        src = SyntheticSource(cfg, int(args.get("--seed", "0")), device, float(args.get("--std", "0.02")))
        recipe = args.get("--recipe", "all")
        tok = ChatTokenizer(build_byte_tokenizer(), DEFAULT_TEMPLATE)
    max_seq = min(max_seq, cfg.max_position_embeddings)
    t_build = time.time()
    w = ModelBuilder(cfg, src, recipe=recipe, device=device, tp_rank=rank if tp > 1 and not cpu else 0,
                     tp_world=tp if not cpu else 1).build()
    if "--model-dir" in args:
        from .checkpoint.io import load_report
        if not cpu:
            torch.cuda.synchronize()
        print(load_report(src, time.time() - t_build), file=sys.stderr)
        if hasattr(src, "close"):
            src.close()
    if cpu:
        from .models.oracle import OracleModel
        runner = OracleModel(w)
    else:
        from .models.runtime import GpuModel
        runner = GpuModel(w, device=device, max_cols=max(16, max_batch), comm=comm)
    return runner, tok, cfg, max_seq


def calib_cache_path(args: Dict[str, str]) -> str:
    base = args.get("--model-dir") or args.get("--synthetic", "tiny")
    key = base.replace("/", "_")
    return os.path.join(os.path.expanduser("~"), ".cache", "velogb10_b200", f"mtp_calib_{key}.json")


def run_server(args: Dict[str, str]):
    import uvicorn
    from .engine.mtp import MtpPolicy
    from .engine.scheduler import Scheduler
    from .server.api import AppState, EngineLoop, create_app
    max_batch = int(args.get("--max-batch", "8"))
    max_seq = int(args.get("--max-seq-len", "4096"))
    t0 = time.time()
    runner, tok, cfg, max_seq = load_runner(args, max_batch, max_seq)
    print(f"[load] total {time.time() - t0:.1f}s model {cfg.name} max_seq_len {max_seq}", file=sys.stderr)
    has_mtp = runner.w.mtp is not None
    r_table = None
    cache = calib_cache_path(args)
    if os.path.exists(cache):
        try:
            r_table = {int(k): float(v) for k, v in json.load(open(cache)).items()}
        except Exception:  # noqa: BLE001 - a corrupt cache only costs a recalibration
            r_table = None
    depth = int(args["--mtp-depth"]) if "--mtp-depth" in args else None
    policy = MtpPolicy(args.get("--mtp", "auto") if has_mtp else "off", depth, r_table, has_head=has_mtp)
    eos = set(tok.stop_token_ids()) | {cfg.eos_token_id}
    sched = Scheduler(runner, max_batch, max_seq, eos_ids=sorted(eos), policy=policy,
                      prefix_cache=on(args.get("--prefix-cache"), True), ngram_draft=int(args.get("--ngram-draft", "0")),
                      tree_draft=on(args.get("--tree-draft"), False), mtp_lanes=on(args.get("--mtp-lanes"), False),
                      zero_kv="--zero-kv" in args, use_graphs="--no-decode-graphs" not in args, log_stream=sys.stderr)
    if has_mtp and r_table is None and policy.mode == "auto" and hasattr(runner, "time_decode_steps"):
        from .gates import calibrate_mtp_r
        try:
            table = calibrate_mtp_r(runner, sched)
            policy.r = table
            os.makedirs(os.path.dirname(cache), exist_ok=True)
            json.dump(table, open(cache, "w"))
        except Exception as e:  # noqa: BLE001
            print(f"[mtp] calibration skipped: {e}", file=sys.stderr)
    name = derive_model_name(args)
    presence = float(args.get("--default-presence-penalty", "2.0" if "2b" in name.lower() else "1.5"))
    rank, world, _ = dist_env()
    lockstep = None
    if world > 1:
        from .parallel.lockstep import Lockstep, run_mirror
        if rank != 0:
            # non-zero ranks replay rank 0's scheduling decisions and never open a port
            run_mirror(sched)
            return
        lockstep = Lockstep(sched)
    engine = EngineLoop(sched, lockstep)
    engine.start()
    state = AppState(engine, tok, name, max_seq, int(args.get("--max-tokens", "8192")),
                     float(args.get("--default-repetition-penalty", "1.0")), presence,
                     float(args.get("--default-frequency-penalty", "0.0")), args.get("--reasoning-effort"))
    app = create_app(state)

    @app.on_event("shutdown")
    def _stop():
        engine.stop()

    def watchdog():
        # the API dies with the scheduler: a dead engine must not keep accepting requests
        while engine.thread.is_alive():
            time.sleep(0.5)
        if engine.error is not None:
            print(f"[server] scheduler died: {engine.error}", file=sys.stderr)
            os._exit(70)

    import threading
    threading.Thread(target=watchdog, daemon=True).start()
    uvicorn.run(app, host=args.get("--host", "0.0.0.0"), port=int(args.get("--port", "8000")), log_level="warning")


def run_generate(args: Dict[str, str]):
    from .engine.mtp import MtpPolicy
    from .engine.sampling import SamplingParams
    from .engine.scheduler import Request, Scheduler
    max_new = int(args.get("--max-new", "32"))
    runner, tok, cfg, max_seq = load_runner(args, 1, int(args.get("--max-seq-len", "4096")))
    if "--prompt-ids" in args:
        ids = [int(x) for x in args["--prompt-ids"].split(",")]
    else:
        ids = tok.encode(args.get("--prompt", "Hello"))
    has_mtp = runner.w.mtp is not None
    sched = Scheduler(runner, 1, max_seq, eos_ids=[cfg.eos_token_id],
                      policy=MtpPolicy(args.get("--mtp", "off") if has_mtp else "off", has_head=has_mtp))
    out: List[int] = []
    t0 = time.time()
    sched.submit(Request(ids, max_new, SamplingParams(temperature=float(args.get("--temperature", "0"))), on_token=out.append))
    sched.run_until_idle()
    dt = time.time() - t0
    print(json.dumps({"tokens": out, "text": tok.decode(out), "tok_per_s": len(out) / dt}))


def run_quantize(args: Dict[str, str]):
    from .checkpoint import io
    stats = io.quantize_checkpoint(args["--model-dir"], args["--out"], args.get("--recipe", "all,gdn:fp8"))
    print(json.dumps(stats))


def run_requant(args: Dict[str, str]):
    from .checkpoint import io
    print(json.dumps(io.requant_gdn(args["--from"], args["--out"])))


def main(argv: Optional[List[str]] = None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    args = parse_args(argv)
    if not args or "--help" in args or "-h" in args:
        print(HELP)
        return 0
    env_bridge(args)
    if "--server" in args:
        run_server(args)
    elif "--quantize" in args:
        run_quantize(args)
    elif "--requant-gdn" in args:
        run_requant(args)
    elif "--generate" in args:
        run_generate(args)
    else:
        from . import gates
        return gates.dispatch(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
