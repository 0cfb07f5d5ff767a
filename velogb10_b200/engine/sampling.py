"""Sampling: seedable host RNG, penalties, nucleus construction and the speculative accept rules.

Numeric contract (reference: kernels/gpu_batch.cu:877-903, :2206-2272, :2483-2600; src/batch.rs:337-360,
:1992-2051):

* greedy when ``temperature < 1e-6``; top-k clamped to [1, 64] and picked by repeated arg-max (lowest
  index wins ties); softmax over the temperature-scaled top-k; nucleus = smallest prefix whose mass
  reaches ``top_p``; draws scale ``u`` by the nucleus mass;
* penalties over the last <= 64 distinct tokens (counts from a <= 256-token history): repetition divides
  positive / multiplies negative logits, presence subtracts a flat amount, frequency ``amount * count``;
* host RNG ``splitmix64(key ^ domain ^ idx * 0x9E3779B97F4A7C15)`` with separate domains for verify,
  accept and sample draws; the key advances once per step;
* stochastic verify with greedy drafts (q = 1): accept draft iff ``u < p(draft)``; on rejection sample from
  the nucleus with the draft's mass removed (full nucleus if nothing is left); a bonus token comes from
  the full nucleus of the last accepted column.

Works on CPU tensors (oracle backend) and on CUDA tensors (device kernels build the nucleus; only the
<= 64 survivors per column travel to the host).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

MASK64 = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15
DOMAIN_VERIFY, DOMAIN_ACCEPT, DOMAIN_SAMPLE = 0x5645524946590000, 0x4143434550540000, 0x53414D504C450000
MAX_TOPK = 64
MAX_PENALTY_TOKENS = 64
HISTORY_CAP = 256


def splitmix64(x: int) -> int:
    x = (x + GOLDEN) & MASK64
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    return z ^ (z >> 31)


def rng_u32(key: int, domain: int, idx: int) -> int:
    return splitmix64((key ^ domain ^ ((idx * GOLDEN) & MASK64)) & MASK64) >> 32


def rng_uniform(key: int, domain: int, idx: int) -> float:
    """Uniform in [0, 1) with 24 bits, the resolution the device sampler uses."""
    return (rng_u32(key, domain, idx) >> 8) / float(1 << 24)


def hash_tokens(tokens: Sequence[int]) -> int:
    """Default request seed: FNV-1a over the prompt ids."""
    h = 0xCBF29CE484222325
    for t in tokens:
        for b in int(t).to_bytes(4, "little"):
            h = ((h ^ b) * 0x100000001B3) & MASK64
    return h


def lcg_uniform(seed: int) -> float:
    """The device sampler's draw: one LCG step, top 24 bits."""
    s = (seed * 1664525 + 1013904223) & 0xFFFFFFFF
    return (s >> 8) / float(1 << 24)


@dataclass
class SamplingParams:
    temperature: float = 0.7
    top_p: float = 0.8
    top_k: int = 20
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: Optional[int] = None

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-6

    @property
    def has_penalty(self) -> bool:
        return self.repetition_penalty != 1.0 or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0


def penalty_list(history: Sequence[int]) -> Tuple[List[int], List[int]]:
    """Last <= 64 distinct tokens of the history (most recent first) with their counts."""
    counts: Dict[int, int] = {}
    for t in history:
        counts[t] = counts.get(t, 0) + 1
    toks: List[int] = []
    seen = set()
    for t in reversed(history):
        if t not in seen:
            seen.add(t)
            toks.append(t)
            if len(toks) == MAX_PENALTY_TOKENS:
                break
    return toks, [counts[t] for t in toks]


def apply_penalties(logits: torch.Tensor, history: Sequence[int], p: SamplingParams) -> torch.Tensor:
    """Penalised copy of one row of logits (any device)."""
    if not p.has_penalty or not history:
        return logits
    toks, cnts = penalty_list(history)
    idx = torch.tensor(toks, dtype=torch.long, device=logits.device)
    v = logits[idx].float()
    if p.repetition_penalty != 1.0:
        v = torch.where(v > 0, v / p.repetition_penalty, v * p.repetition_penalty)
    v = v - p.presence_penalty - p.frequency_penalty * torch.tensor(cnts, dtype=torch.float32, device=logits.device)
    out = logits.clone()
    out[idx] = v.to(out.dtype)
    return out


@dataclass
class Nucleus:
    ids: List[int]
    probs: List[float]          # softmax over the scaled top-k (not renormalised to the nucleus)

    @property
    def mass(self) -> float:
        return float(sum(self.probs))

    def prob_of(self, tok: int) -> float:
        """Probability of ``tok`` under the renormalised nucleus."""
        for i, p in zip(self.ids, self.probs):
            if i == tok:
                return p / self.mass
        return 0.0

    def draw(self, u: float) -> int:
        target = u * self.mass
        c = 0.0
        for i, p in zip(self.ids, self.probs):
            c += p
            if target < c:
                return i
        return self.ids[-1]

    def without(self, tok: int) -> "Nucleus":
        ids = [i for i in self.ids if i != tok]
        probs = [p for i, p in zip(self.ids, self.probs) if i != tok]
        if not ids or sum(probs) <= 0.0:
            return self
        return Nucleus(ids, probs)


def nucleus_host(logits: torch.Tensor, p: SamplingParams) -> Nucleus:
    """Reference implementation on a CPU row of logits."""
    lf = logits.float()
    if p.greedy:
        return Nucleus([_argmax_low(lf)], [1.0])
    k = max(1, min(MAX_TOPK, int(p.top_k)))
    k = min(k, lf.numel())
    vals, idx = torch.sort(lf, descending=True, stable=True)     # stable: lowest index first among ties
    vals, idx = vals[:k], idx[:k]
    sc = vals / p.temperature
    e = torch.exp(sc - sc[0])
    pr = (e / e.sum()).tolist()
    keep, cum = k, 0.0
    for r in range(k):
        cum += pr[r]
        if cum >= p.top_p:
            keep = r + 1
            break
    return Nucleus(idx[:keep].tolist(), pr[:keep])


def _argmax_low(row: torch.Tensor) -> int:
    m = row.max()
    return int(torch.nonzero(row == m)[0])


def nucleus_rows(logits: torch.Tensor, params: Sequence[SamplingParams]) -> List[Nucleus]:
    """Nucleus per row of ``logits`` [N, V]; uses the device kernel for CUDA tensors."""
    n = logits.shape[0]
    if not logits.is_cuda:
        return [nucleus_host(logits[i], params[i]) for i in range(n)]
    from ..ops import kernels as K
    dev = logits.device
    temp = torch.tensor([p.temperature for p in params], dtype=torch.float32, device=dev)
    tk = torch.tensor([p.top_k for p in params], dtype=torch.int32, device=dev)
    tp = torch.tensor([p.top_p for p in params], dtype=torch.float32, device=dev)
    ids = torch.empty((n, MAX_TOPK), dtype=torch.int32, device=dev)
    probs = torch.empty((n, MAX_TOPK), dtype=torch.float32, device=dev)
    keep = torch.empty((n,), dtype=torch.int32, device=dev)
    lg = logits if logits.dtype == torch.float32 else logits.float()
    K.nucleus(lg, n, temp, tk, tp, None, None, ids, probs, keep)
    ids_h, probs_h, keep_h = ids.cpu(), probs.cpu(), keep.cpu().tolist()
    return [Nucleus(ids_h[i, :keep_h[i]].tolist(), probs_h[i, :keep_h[i]].tolist()) for i in range(n)]


def argmax_rows(logits: torch.Tensor) -> List[int]:
    """Greedy token per row, lowest index on ties."""
    if logits.is_cuda and logits.dtype == torch.float32:
        from ..ops import kernels as K
        out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
        K.argmax(logits, logits.shape[0], out)
        return out.tolist()
    return [_argmax_low(logits[i].float()) for i in range(logits.shape[0])]


# ------------------------------------------------------------------ speculative accept rules

def greedy_accept(preds: Sequence[int], drafts: Sequence[int]) -> int:
    """Length of the longest prefix of ``drafts`` the target agrees with (preds[t] follows column t)."""
    n = 0
    while n < len(drafts) and preds[n] == drafts[n]:
        n += 1
    return n


def tree_accept_walk(parent: Sequence[int], tokens: Sequence[int], preds: Sequence[int]) -> List[int]:
    """Follow the target's arg-max down a draft tree. Column 0 is the root (already committed token);
    returns the accepted column path starting with 0. A child is taken when its token equals the
    prediction of the current node; among equal children the lowest column wins
    (reference: src/batch.rs:380-398)."""
    path = [0]
    cur = 0
    while True:
        nxt = -1
        for c in range(cur + 1, len(tokens)):
            if parent[c] == cur and tokens[c] == preds[cur]:
                nxt = c
                break
        if nxt < 0:
            return path
        path.append(nxt)
        cur = nxt


def stochastic_accept(nuclei: Sequence[Nucleus], drafts: Sequence[int], key: int) -> Tuple[int, int]:
    """Distribution-exact acceptance of greedy drafts. Returns (n_accepted, next_token) where
    next_token is the residual resample at the first rejection or the bonus draw after full acceptance."""
    for t, d in enumerate(drafts):
        p = nuclei[t].prob_of(d)
        u = rng_uniform(key, DOMAIN_ACCEPT, t)
        if u < p:
            continue
        res = nuclei[t].without(d)
        return t, res.draw(rng_uniform(key, DOMAIN_VERIFY, t))
    t = len(drafts)
    return t, nuclei[t].draw(rng_uniform(key, DOMAIN_VERIFY, t))
