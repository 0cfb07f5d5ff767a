"""Self-tuning policy for multi-token-prediction (MTP) speculative decoding.

``speedup(d) = yield(d) / r(d)``: ``yield`` is the expected number of tokens emitted per speculative
step at draft depth ``d`` estimated from per-position acceptance hazards, ``r(d)`` the measured cost of
one draft+verify(+reprime+rollback) step relative to a plain decode step. Every ``WINDOW`` speculative
steps the policy moves to the best calibrated depth if it wins by ``MARGIN``, switches speculation off
when no depth beats plain decoding and probes again after ``RETRY`` plain steps
(reference: src/batch.rs:118-318, depth set src/gpu.rs:186-188).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

AUTO_DEPTHS = (2, 3, 4, 5, 6, 8)
WINDOW = 128
MARGIN = 1.05
RETRY = 4096
START_DEPTH = 4
MIN_OBS = 8
PRIOR = 0.5
MAX_DEPTH = 16

# cost ratios used until a calibration run provides measured ones (a verify of width d costs little more
# than a decode because the GEMMs are weight-bandwidth bound and flat in the width)
DEFAULT_R = {2: 1.15, 3: 1.22, 4: 1.30, 5: 1.38, 6: 1.46, 8: 1.62}


class MtpPolicy:
    def __init__(self, mode: str = "auto", depth: Optional[int] = None, r: Optional[Dict[int, float]] = None,
                 has_head: bool = True):
        assert mode in ("auto", "on", "off")
        self.mode = mode
        self.r = dict(DEFAULT_R if r is None else r)
        self.fixed_depth = depth
        self.depth = depth if depth else START_DEPTH
        self.active = has_head and mode != "off"
        self.has_head = has_head
        self.tried = [0] * MAX_DEPTH
        self.acc = [0] * MAX_DEPTH
        self.steps_in_window = 0
        self.plain_steps = 0
        self.total_steps = 0
        self.total_emitted = 0
        self.total_drafts = 0
        self.total_accepted = 0
        self.log: List[str] = []

    # ---- statistics
    def record_step(self, drafts: int, accepted: int, emitted: int):
        for j in range(min(drafts, MAX_DEPTH)):
            self.tried[j] += 1
            if j < accepted:
                self.acc[j] += 1
        self.total_steps += 1
        self.total_emitted += emitted
        self.total_drafts += drafts
        self.total_accepted += accepted
        self.steps_in_window += 1
        if self.steps_in_window >= WINDOW:
            self._retune()

    def hazard(self, j: int) -> float:
        """Acceptance probability of draft position j given positions < j were accepted."""
        last = PRIOR
        for i in range(j + 1):
            # position i is only tried when i-1 was accepted, so the conditional rate is acc[i] / acc[i-1]
            base = self.tried[0] if i == 0 else self.acc[i - 1]
            if base >= MIN_OBS:
                last = self.acc[i] / base
        return last

    def yield_at(self, depth: int) -> float:
        """Expected tokens emitted per step with ``depth`` verify columns (depth-1 drafts + 1 bonus)."""
        y, surv = 1.0, 1.0
        for j in range(depth - 1):
            surv *= self.hazard(j)
            y += surv
        return y

    def score(self, depth: int) -> float:
        return self.yield_at(depth) / self.r.get(depth, DEFAULT_R.get(depth, 1.0 + 0.08 * depth))

    # ---- control
    def _retune(self):
        self.steps_in_window = 0
        if self.mode != "auto":
            return
        cands = [d for d in AUTO_DEPTHS if d in self.r]
        best = max(cands, key=self.score)
        if self.fixed_depth is None and best != self.depth and self.score(best) > self.score(self.depth) * MARGIN:
            self.log.append(f"[mtp] depth {self.depth} -> {best} (score {self.score(best):.3f})")
            self.depth = best
        if self.score(self.depth if self.fixed_depth else best) < 1.0:
            self.active = False
            self.plain_steps = 0
            self.log.append(f"[mtp] disabled (best score {self.score(best):.3f} < 1)")

    def tick(self):
        """Called once per scheduler step; re-arms speculation after RETRY plain steps."""
        if self.mode == "auto" and self.has_head and not self.active:
            self.plain_steps += 1
            if self.plain_steps >= RETRY:
                self.active = True
                self.tried = [0] * MAX_DEPTH
                self.acc = [0] * MAX_DEPTH
                self.log.append("[mtp] re-probing")

    def acceptance(self) -> float:
        return self.total_accepted / self.total_drafts if self.total_drafts else 0.0

    def accept_curve(self) -> List[dict]:
        """Cumulative accept-by-depth curve: per draft position its accepted / offered counts, their ratio and the
        chance that a draft chain reaches that depth (the product of the rates so far), which is what drives the
        yield (reference: src/batch.rs:1717-1741 ``dump_accept_curve``)."""
        out, chain = [], 1.0
        for j in range(MAX_DEPTH):
            if not self.tried[j]:
                break
            rate = self.acc[j] / self.tried[j]
            chain *= rate
            out.append({"pos": j + 1, "accepted": self.acc[j], "offered": self.tried[j], "rate": rate, "cond_chain": chain})
        return out

    def curve(self) -> List[float]:
        return [self.acc[j] / self.tried[j] if self.tried[j] else 0.0 for j in range(8)]
