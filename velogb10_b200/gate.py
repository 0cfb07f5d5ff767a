"""Statistical gate runner: loops the randomized gates of ``velogb10_b200.gates`` until a sequential
probability ratio test decides, and charts benchmark metrics against a frozen baseline.

  python -m velogb10_b200.gate --synthetic tiny --cpu            # all gates, SPRT over randomized draws
  python -m velogb10_b200.gate --model-dir DIR --history gate_history.csv

Design rules carried over from the reference runner (reference: scripts/gate.py:9-55, :206-211): a gate
loops over randomized draws with a stopping rule instead of running once; a check must prove it extracted
something (a missing value is "could not measure", exit code 2, never a pass); metric drift is judged with
a Shewhart 3-sigma rule and a CUSUM (k = 0.5, h = 5) against the first 8 green runs.
Exit codes: 0 pass, 1 fail, 2 could not measure.
"""
from __future__ import annotations

import csv
import json
import math
import os
import subprocess
import sys
from typing import Dict, List, Optional, Tuple

P0, P1, ALPHA, BETA = 0.001, 0.3, 0.01, 0.01
BASELINE_RUNS = 8


def sprt_bounds(alpha: float = ALPHA, beta: float = BETA) -> Tuple[float, float]:
    return math.log(beta / (1 - alpha)), math.log((1 - beta) / alpha)


def sprt_update(llr: float, failed: bool, p0: float = P0, p1: float = P1) -> float:
    return llr + (math.log(p1 / p0) if failed else math.log((1 - p1) / (1 - p0)))


def sprt(draw, max_draws: int = 200) -> Tuple[str, int]:
    """Runs ``draw(i) -> True (clean) / False (failure) / None (could not measure)`` until a decision."""
    lo, hi = sprt_bounds()
    llr = 0.0
    for i in range(max_draws):
        r = draw(i)
        if r is None:
            return "unmeasured", i + 1
        llr = sprt_update(llr, not r)
        if llr <= lo:
            return "pass", i + 1
        if llr >= hi:
            return "fail", i + 1
    return "undecided", max_draws


def extract(line: str, key: str):
    """Value of ``key`` in a JSON gate line; raises when absent so a silent gate cannot pass."""
    d = json.loads(line)
    if key not in d:
        raise KeyError(f"{key} missing from gate output")
    return d[key]


def shewhart_cusum(history: List[float], value: float, k: float = 0.5, h: float = 5.0) -> Dict[str, object]:
    base = history[:BASELINE_RUNS]
    if len(base) < BASELINE_RUNS:
        return {"status": "collecting", "n": len(base)}
    mu = sum(base) / len(base)
    sd = math.sqrt(sum((x - mu) ** 2 for x in base) / (len(base) - 1)) or 1e-9
    z = (value - mu) / sd
    cp = cm = 0.0
    for x in history[BASELINE_RUNS:] + [value]:
        zx = (x - mu) / sd
        cp = max(0.0, cp + zx - k)
        cm = max(0.0, cm - zx - k)
    return {"status": "drift" if abs(z) > 3 or cp > h or cm > h else "ok", "z": z, "cusum_hi": cp, "cusum_lo": cm}


def run_gate(base_args: List[str], mode: str, extra: List[str]) -> Optional[dict]:
    cmd = [sys.executable, "-m", "velogb10_b200", mode] + base_args + extra
    r = subprocess.run(cmd, capture_output=True, text=True)
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    if not lines:
        return None
    try:
        return json.loads(lines[-1])
    except json.JSONDecodeError:
        return None


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    history_path = None
    if "--history" in argv:
        i = argv.index("--history")
        history_path = argv[i + 1]
        argv = argv[:i] + argv[i + 2:]
    results = {}

    def verify_draw(i):
        out = run_gate(argv, "--bench-verify", ["--draws", "2", "--seed", str(i)])
        return None if out is None or "pass" not in out else bool(out["pass"])

    results["verify-fuzz"] = sprt(verify_draw, 40)
    for mode in ("--probe-binv", "--probe-state", "--bench-tree", "--bench-lanes", "--bench-mtp"):
        out = run_gate(argv, mode, [])
        results[mode] = ("unmeasured", 1) if out is None or "pass" not in out else (("pass" if out["pass"] else "fail"), 1)
    perf = run_gate(argv, "--bench-batch", [])
    drift = None
    if perf is not None and history_path:
        hist: List[float] = []
        if os.path.exists(history_path):
            with open(history_path) as f:
                hist = [float(r["tok_s"]) for r in csv.DictReader(f)]
        drift = shewhart_cusum(hist, float(extract(json.dumps(perf), "tok_s")))
        green = all(v[0] == "pass" for v in results.values())
        if green:
            new = not os.path.exists(history_path)
            with open(history_path, "a", newline="") as f:
                w = csv.writer(f)
                if new:
                    w.writerow(["tok_s"])
                w.writerow([perf["tok_s"]])
    print(json.dumps({"gates": {k: {"verdict": v[0], "draws": v[1]} for k, v in results.items()}, "drift": drift}))
    verdicts = [v[0] for v in results.values()]
    if "fail" in verdicts or (drift and drift.get("status") == "drift"):
        return 1
    if "unmeasured" in verdicts or "undecided" in verdicts:
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
