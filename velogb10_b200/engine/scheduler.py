"""Continuous-batching scheduler with slot indirection, per-slot prefix cache (live and prompt
checkpoints), chunked prefill, and MTP speculative decoding (greedy chain, stochastic chain, n-gram fork
tree, multi-lane forest).

Behavioural spec (reference: src/batch.rs:400-531 state, :750-771 loop, :954-1153 admission,
:1160-1285 decode step, :1390-1523 tree, :1534-1698 forest, :1743-1949 greedy chain, :1959-2147
stochastic chain, :2153-2267 batched decode):

* lanes are front-packed logical positions; each holds a physical slot into the KV / recurrent-state store;
  finishing a lane returns the slot without copying state, and the slot keeps its token list for reuse;
* admission picks, among free slots, the longest cached sequence (live state or prompt checkpoint) that is
  a strict prefix of the prompt, prefills the remainder in windows with a forced boundary at the chat
  template's checkpoint position, primes the draft head, and emits the first token immediately;
* a decode step runs phase A (speculation: one lane, or a packed forest of greedy lanes) then phase B
  (one batched decode over the remaining lanes);
* greedy speculation is exactly lossless because a width-N verify is bit-identical to N decodes.

The scheduler drives any *runner* exposing ``prefill / decode / verify / verify_forest / mtp_forward /
copy_state / zero_slot / compact_kv`` (the CUDA runtime or the fp32 CPU oracle).
"""
from __future__ import annotations

import json
import os
import sys
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence, Set, Tuple

import torch

from . import sampling as S
from .mtp import MtpPolicy
from .sampling import SamplingParams

PREFILL_WINDOW = 8192
MTP_PRIME_CHUNK = 2048
VERIFY_CKPTS = 17            # 16 verify columns + 1 scratch (tree root)
class _phase:
    """NVTX range around a scheduler phase (``VELO_NVTX=1``), so a timeline profiler shows admission / prefill and
    decode steps as named spans; a no-op otherwise."""

    def __init__(self, name: str, on: bool):
        self.name, self.on = name, on

    def __enter__(self):
        if self.on:
            import torch
            torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        if self.on:
            import torch
            torch.cuda.nvtx.range_pop()
        return False


MTP_LOG_EVERY = 50
MAX_FOREST_LANES = 5
MAX_VERIFY_COLS = 16


@dataclass
class Request:
    prompt: List[int]
    max_new_tokens: int = 256
    params: SamplingParams = field(default_factory=SamplingParams)
    stop_ids: Set[int] = field(default_factory=set)
    ckpt_at: Optional[int] = None                     # prompt position of the chat-template boundary
    on_token: Optional[Callable[[int], None]] = None
    on_finish: Optional[Callable[[str, dict], None]] = None
    id: int = 0
    cancelled: bool = False                           # set by the owner of the request at any time (any thread)
    cancel_applied: bool = False                      # set by the scheduler at a step boundary; the only flag it acts on
    # filled by the scheduler
    t_submit: float = 0.0
    t_first: float = 0.0
    prefix_hit: int = 0


@dataclass
class Lane:
    req: Request
    slot: int
    pos: int                     # tokens whose state lives in the slot == next feed position
    last_tok: int                # emitted but not yet fed
    generated: int
    history: List[int]
    key: int                     # RNG state, advances once per step
    h_prev: Optional[torch.Tensor] = None      # backbone hidden that predicted last_tok (draft head input)
    mtp_ok: bool = False
    done: Optional[str] = None


class Scheduler:
    def __init__(self, runner, max_batch: int, max_seq: int, eos_ids: Sequence[int] = (), policy: Optional[MtpPolicy] = None,
                 prefix_cache: bool = True, ngram_draft: int = 0, tree_draft: bool = False, mtp_lanes: bool = False,
                 prefill_window: int = PREFILL_WINDOW, zero_kv: bool = False, use_graphs: bool = True,
                 alloc: bool = True, log_stream=None):
        self.r = runner
        # Log lines ([req] admission / completion, [mtp] policy moves and the periodic acceptance line) are kept in a
        # bounded ring and, when a stream is given (the server passes stderr), written as they happen
        # (reference: src/batch.rs:1002-1005, :1059-1061, :294-315, :1936-1947).
        self.log_stream = log_stream
        self.log: Deque[str] = deque(maxlen=4096)
        # VELO_MTP_DRAFT_LOG=path: one JSON object per chain-MTP step {step, lane, pos, committed, drafts, preds, nacc}
        # (preds empty where the verify samples); VELO_MTP_CURVE_FILE=path: cumulative accept-by-depth curve,
        # rewritten every MTP_LOG_EVERY speculative steps (reference: src/batch.rs:520-527, :1700-1741).
        self._draft_log = None
        path = os.environ.get("VELO_MTP_DRAFT_LOG")
        if path:
            try:
                self._draft_log = open(path, "w")
            except OSError as e:
                print(f"[mtp] cannot open VELO_MTP_DRAFT_LOG {path}: {e}", file=sys.stderr)
        self._curve_path = os.environ.get("VELO_MTP_CURVE_FILE")
        self.max_batch, self.max_seq = max_batch, max_seq
        self.eos = set(int(e) for e in eos_ids)
        self.has_mtp = getattr(runner, "w", None) is not None and runner.w.mtp is not None
        self.policy = policy or MtpPolicy("auto" if self.has_mtp else "off", has_head=self.has_mtp)
        self.prefix_cache = prefix_cache
        self.ngram, self.tree, self.mtp_lanes = ngram_draft, tree_draft, mtp_lanes
        self.nvtx = os.environ.get("VELO_NVTX", "0") == "1" and hasattr(runner, "dev")
        if hasattr(runner, "tc_decode_attn"):
            # Tree verification needs the path-indirect attention kernel; a tree column equals the same column of a
            # chain verify bit for bit only if chains and decodes take that kernel too, so tree drafting turns the
            # tensor-core decode attention off for this runner (and a scheduler without it restores the default).
            want = runner.tc_decode_attn_default and not (tree_draft and ngram_draft > 0)
            if want != runner.tc_decode_attn:
                runner.tc_decode_attn = want
                runner.graphs.clear()                      # captured steps hold the other kernel
        self.window = prefill_window
        self.zero_kv = zero_kv
        self.use_graphs = use_graphs and hasattr(runner, "replay_decode")
        # state-slot map: [0, B) lanes | [B, B+17) verify checkpoints | [B+17, 2B+17) prompt checkpoints
        self.ckpt_base = max_batch
        self.prompt_ckpt_base = max_batch + VERIFY_CKPTS
        if alloc:
            runner.alloc_state(max_batch, 2 * max_batch + VERIFY_CKPTS, max_seq)
        self.free_slots: List[int] = list(range(max_batch))
        self.slot_cache: List[List[int]] = [[] for _ in range(max_batch)]
        self.slot_ckpt_seq: List[List[int]] = [[] for _ in range(max_batch)]
        self.lanes: List[Lane] = []
        self.queue: Deque[Request] = deque()
        self.next_id = 1
        self.stats = {"admitted": 0, "prefix_live": 0, "prefix_ckpt": 0, "prefix_miss": 0, "decode_steps": 0,
                      "mtp_steps": 0, "forest_steps": 0, "tree_steps": 0, "tokens": 0, "prefill_tokens": 0}
        # True when something else (the lockstep driver) decides which cancellations a step sees, so that every
        # rank of a tensor-parallel group applies the same ones in the same step
        self.external_cancels = False
        # optional health probe called once per step; raises when a kernel or a collective reported a failure
        self.health_check: Optional[Callable[[], None]] = getattr(runner, "health_check", None)
        # wall time of the most recent decode steps (ms), for per-token latency percentiles; --tp-trace prints them
        self.step_ms: Deque[float] = deque(maxlen=4096)
        self.trace_every = 256 if os.environ.get("VELO_TP_TRACE", "0") == "1" else 0
        self.cpu_sample = os.environ.get("VELO_CPU_SAMPLE", "0") == "1"
        # token selection on the device when the runner has a sampler (--cpu-sample forces the host path): forwards
        # then return this rank's vocabulary shard and full logits never leave the GPU or cross ranks
        self.sampler = None if self.cpu_sample else getattr(runner, "sampler", None)
        if self.sampler is not None:
            runner.gather_logits = False

    # ------------------------------------------------------------------ public
    def submit(self, req: Request) -> int:
        req.id = self.next_id
        self.next_id += 1
        req.t_submit = time.time()
        self.queue.append(req)
        return req.id

    def idle(self) -> bool:
        return not self.lanes and not self.queue

    def run_until_idle(self, max_steps: int = 1 << 30):
        n = 0
        while not self.idle() and n < max_steps:
            self.step()
            n += 1

    def apply_cancels(self, ids: Optional[Set[int]] = None):
        """Latch cancellations at a step boundary. ``ids=None`` snapshots the live ``cancelled`` flags of every
        running and queued request; otherwise exactly the requests named are cancelled (lockstep: the head's
        snapshot, replayed identically on every rank). The step acts on the latched flag only, so a flag that
        flips while the step runs is seen by the next one."""
        for req in [l.req for l in self.lanes] + list(self.queue):
            if (req.cancelled if ids is None else req.id in ids):
                req.cancel_applied = True

    def pending_cancels(self) -> List[int]:
        """Ids of running or queued requests whose owner cancelled them and that no step has acted on yet."""
        return [r.id for r in [l.req for l in self.lanes] + list(self.queue) if r.cancelled and not r.cancel_applied]

    def _log(self, line: str):
        self.log.append(line)
        if self.log_stream is not None:
            print(line, file=self.log_stream, flush=True)

    def _log_mtp_step(self, lane: "Lane", pos: int, committed: int, drafts: Sequence[int], preds: Sequence[int], nacc: int):
        """Book-keeping after a speculative step of one lane: the draft log line, the policy's own messages, and every
        MTP_LOG_EVERY steps the acceptance line with the accept-by-depth curve (also written to the curve file)."""
        step = self.stats["mtp_steps"]
        if self._draft_log is not None:
            self._draft_log.write(json.dumps({"step": step, "lane": lane.slot, "pos": pos, "committed": int(committed),
                                              "drafts": [int(x) for x in drafts], "preds": [int(x) for x in preds],
                                              "nacc": int(nacc)}) + "\n")
            self._draft_log.flush()
        while self.policy.log:
            self._log(self.policy.log.pop(0))
        if step and step % MTP_LOG_EVERY == 0:
            pol = self.policy
            curve = pol.accept_curve()
            self._log(f"[mtp] steps {step} depth {pol.depth} acceptance {pol.acceptance():.3f} tokens/step "
                       f"{pol.total_emitted / max(1, pol.total_steps):.2f} accept@k "
                       + " ".join(f"{c['rate']:.2f}" for c in curve[:pol.depth - 1]))
            if self._curve_path:
                try:
                    with open(self._curve_path, "w") as f:
                        json.dump({"depth": pol.depth, "steps": step, "accept_by_depth": curve}, f)
                except OSError:
                    pass

    def step(self) -> bool:
        """Admit what fits, then run one decode step. Returns False when there was nothing to do."""
        if not self.external_cancels:
            self.apply_cancels(None)
        if self.health_check is not None:
            self.health_check()
        with _phase("admit + prefill", self.nvtx and bool(self.queue)):
            while self.queue and self.free_slots and len(self.lanes) < self.max_batch:
                self._admit(self.queue.popleft())
        if not self.lanes:
            return False
        t0 = time.perf_counter()
        with _phase(f"decode step, {len(self.lanes)} lanes", self.nvtx):
            self._decode_step()
        self.step_ms.append((time.perf_counter() - t0) * 1e3)
        if self.trace_every and len(self.step_ms) % self.trace_every == 0:
            print("[trace] step latency ms " + " ".join(f"{k}={v:.3f}" for k, v in self.latency_percentiles().items()),
                  file=sys.stderr)
        return True

    def latency_percentiles(self) -> Dict[str, float]:
        """p50 / p90 / p99 / max of the recorded decode-step wall times (reference: src/gpu.rs:7296-7364 reports the
        same percentiles per token)."""
        v = sorted(self.step_ms)
        if not v:
            return {}
        pick = lambda q: v[min(len(v) - 1, int(q * len(v)))]
        return {"n": float(len(v)), "p50": pick(0.50), "p90": pick(0.90), "p99": pick(0.99), "max": v[-1]}

    # ------------------------------------------------------------------ admission
    def _pick_slot(self, prompt: List[int]) -> Tuple[int, int, str]:
        """(slot, reused_len, kind) with kind in live / ckpt / miss."""
        best = (-1, 0, "miss")
        if self.prefix_cache:
            for s in self.free_slots:
                for kind, seq in (("live", self.slot_cache[s]), ("ckpt", self.slot_ckpt_seq[s])):
                    n = len(seq)
                    if 0 < n < len(prompt) and n > best[1] and prompt[:n] == seq:
                        best = (s, n, kind)
        if best[0] < 0:
            # prefer a slot without cached state so cached prefixes survive longer
            empty = [s for s in self.free_slots if not self.slot_cache[s] and not self.slot_ckpt_seq[s]]
            return (empty[0] if empty else self.free_slots[0]), 0, "miss"
        return best

    def _finish_req(self, req: Request, reason: str, prompt_tokens: int, completion: int):
        if req.on_finish:
            now = time.time()
            req.on_finish(reason, {"prompt_tokens": prompt_tokens, "completion_tokens": completion,
                                   "prefix_hit": req.prefix_hit, "t_submit": req.t_submit, "t_first": req.t_first,
                                   "t_done": now})

    def _admit(self, req: Request):
        prompt = list(req.prompt)
        plen = len(prompt)
        if req.cancel_applied:
            self._finish_req(req, "cancelled", plen, 0)
            return
        if plen == 0 or plen >= self.max_seq:
            self._finish_req(req, "context_length_exceeded", plen, 0)
            return
        slot, reuse, kind = self._pick_slot(prompt)
        self.free_slots.remove(slot)
        max_new = max(1, min(req.max_new_tokens, self.max_seq - plen))
        r = self.r
        if kind == "ckpt":
            r.copy_state(self.prompt_ckpt_base + slot, slot)
            self.stats["prefix_ckpt"] += 1
        elif kind == "live":
            self.stats["prefix_live"] += 1
        else:
            r.zero_slot(slot, self.zero_kv)
            self.slot_ckpt_seq[slot] = []
            self.stats["prefix_miss"] += 1
        req.prefix_hit = reuse
        p_ = req.params
        self._log(f"[req] {req.id} slot {slot} prompt {plen} prefix {kind} {reuse} max_new {max_new}"
                   + (f" (clamped from {req.max_new_tokens})" if max_new != req.max_new_tokens else "")
                   + f" temp {p_.temperature} top_p {p_.top_p} top_k {p_.top_k} rep {p_.repetition_penalty} "
                     f"pres {p_.presence_penalty} freq {p_.frequency_penalty}")
        # prefill the suffix in windows; force a window boundary at the checkpoint position
        ckpt_at = req.ckpt_at if (req.ckpt_at is not None and reuse < req.ckpt_at < plen) else None
        pos = reuse
        logits = None
        h_last = None
        did_ckpt = False
        while pos < plen:
            end = min(plen, pos + self.window)
            if ckpt_at is not None and pos < ckpt_at < end:
                end = ckpt_at
            logits, hidden = r.prefill(slot, prompt[pos:end], pos)
            if self.has_mtp and hidden is not None:
                self._mtp_prime(slot, prompt, pos, end, hidden, h_last)
                h_last = hidden[-1].clone()
            self.stats["prefill_tokens"] += end - pos
            pos = end
            if ckpt_at is not None and pos == ckpt_at:
                r.copy_state(slot, self.prompt_ckpt_base + slot)
                self.slot_ckpt_seq[slot] = prompt[:pos]
                did_ckpt = True
        if not did_ckpt and self.prefix_cache and kind != "ckpt":
            r.copy_state(slot, self.prompt_ckpt_base + slot)
            self.slot_ckpt_seq[slot] = prompt[:plen]
        self.slot_cache[slot] = list(prompt)
        key = req.params.seed if req.params.seed is not None else S.hash_tokens(prompt)
        key &= S.MASK64
        first = self._pick_token(logits.reshape(1, -1), [req.params], [[]], [key])[0]
        key = S.splitmix64(key)
        req.t_first = time.time()
        lane = Lane(req, slot, plen, first, 1, [first], key, h_last, self.has_mtp and h_last is not None)
        self.stats["admitted"] += 1
        self.lanes.append(lane)
        self._emit(lane, [first])
        self._retire_finished()

    def _mtp_prime(self, slot, prompt, pos, end, hidden, h_before):
        """Feed (hidden[t], token[t+1]) pairs of this window into the draft head's KV cache."""
        toks, hs, ps = [], [], []
        if h_before is not None and pos > 0:
            toks.append(prompt[pos]); hs.append(h_before); ps.append(pos - 1)
        for t in range(pos, end - 1):
            toks.append(prompt[t + 1]); hs.append(hidden[t - pos]); ps.append(t)
        self._mtp_prime_small(slot, toks, hs, ps)

    def _mtp_prime_small(self, slot, toks, hs, ps):
        for o in range(0, len(toks), MAX_VERIFY_COLS):
            self.r.mtp_forward(slot, toks[o:o + MAX_VERIFY_COLS], torch.stack(hs[o:o + MAX_VERIFY_COLS]),
                               ps[o:o + MAX_VERIFY_COLS])

    # ------------------------------------------------------------------ token selection
    def _pick_token(self, logits: torch.Tensor, params: Sequence[SamplingParams], histories: Sequence[Sequence[int]],
                    keys: Sequence[int]) -> List[int]:
        """One token per row: penalties, then arg-max or a seeded nucleus draw."""
        n = logits.shape[0]
        if self.sampler is not None and logits.is_cuda:
            lg = logits if logits.dtype == torch.float32 else logits.float()
            return self.sampler.pick(lg, list(params), [list(h) for h in histories], list(keys))
        if any(p.has_penalty and h for p, h in zip(params, histories)):
            logits = logits.clone() if logits.dtype == torch.float32 else logits.float()
            for i in range(n):
                if params[i].has_penalty and histories[i]:
                    logits[i] = S.apply_penalties(logits[i], histories[i], params[i])
        if all(p.greedy for p in params):
            return S.argmax_rows(logits if logits.dtype == torch.float32 else logits.float())
        nuclei = S.nucleus_rows(logits, params)
        return [nuc.draw(S.rng_uniform(keys[i], S.DOMAIN_SAMPLE, 0)) for i, nuc in enumerate(nuclei)]

    # ------------------------------------------------------------------ emission / retirement
    def _emit(self, lane: Lane, toks: Sequence[int]):
        """Deliver tokens with the budget and stop-set discipline (applies to accepted drafts too)."""
        req = lane.req
        for t in toks:
            if lane.done:
                break
            if t in self.eos or t in req.stop_ids:
                lane.done = "stop"
                break
            if req.on_token:
                req.on_token(t)
            self.stats["tokens"] += 1
            if lane.generated >= min(req.max_new_tokens, self.max_seq - len(req.prompt)):
                lane.done = "length"
        if lane.pos + 1 >= self.max_seq and not lane.done:
            lane.done = "length"

    def _retire_finished(self):
        keep = []
        for lane in self.lanes:
            if lane.req.cancel_applied and not lane.done:
                lane.done = "cancelled"
            if lane.done:
                self.free_slots.append(lane.slot)
                # a cancelled request still gets its final event: whoever waits on it must be released
                self._finish_req(lane.req, lane.done, len(lane.req.prompt), lane.generated)
                dt = time.time() - lane.req.t_first if lane.req.t_first else 0.0
                self._log(f"[req] {lane.req.id} done {lane.done} generated {lane.generated}"
                           + (f" in {dt:.2f}s ({lane.generated / dt:.1f} tok/s)" if dt > 0 else ""))
            else:
                keep.append(lane)
        self.lanes = keep

    def _push_history(self, lane: Lane, toks: Sequence[int]):
        lane.history.extend(toks)
        if len(lane.history) > S.HISTORY_CAP:
            del lane.history[:S.HISTORY_CAP // 2]

    # ------------------------------------------------------------------ decode step
    def _decode_step(self):
        self._retire_finished()
        if not self.lanes:
            return
        handled: List[Lane] = []
        if self.policy.active and self.has_mtp:
            ready = [l for l in self.lanes if l.mtp_ok]
            if len(self.lanes) == 1 and ready:
                lane = ready[0]
                if lane.req.params.greedy:
                    if self.tree and self.ngram > 0:
                        self._mtp_tree_step(lane)
                    else:
                        self._mtp_chain_step(lane)
                else:
                    self._mtp_sample_step(lane)
                handled.append(lane)
            elif self.mtp_lanes and len(self.lanes) >= 2:
                greedy = [l for l in ready if l.req.params.greedy and not l.req.params.has_penalty][:MAX_FOREST_LANES]
                if len(greedy) >= 2:
                    self._mtp_forest_step(greedy)
                    handled.extend(greedy)
                for l in ready:
                    if l not in handled and not l.req.params.greedy:
                        self._mtp_sample_step(l)
                        handled.append(l)
        self.policy.tick()
        rest = [l for l in self.lanes if l not in handled and not l.done]
        if rest:
            self._batched_decode(rest)
        self._retire_finished()

    def _batched_decode(self, lanes: List[Lane]):
        toks = [l.last_tok for l in lanes]
        pos = [l.pos for l in lanes]
        slots = [l.slot for l in lanes]
        plain = all(l.req.params.greedy and not l.req.params.has_penalty for l in lanes)
        if plain and self.use_graphs:
            # greedy graph; the hidden rows the draft head needs stay in the runner's fixed workspace buffer
            new = self.r.replay_decode(toks, pos, slots).tolist()
            hidden = self.r.ws.x[:len(lanes)] if self.has_mtp else None
            self.stats["graph_steps"] = self.stats.get("graph_steps", 0) + 1
        elif self.use_graphs and self.sampler is not None and hasattr(self.r, "replay_decode_sample"):
            # decode + sample graph: parameters, uniforms and penalty lists go up in one copy, one read comes back
            self.r.ensure_sample_graph(len(lanes))
            params = [l.req.params for l in lanes]
            u = [S.rng_uniform(l.key, S.DOMAIN_SAMPLE, 0) for l in lanes]
            self.sampler.upload(params, u=u, histories=[l.history for l in lanes])
            new = self.r.replay_decode_sample(toks, pos, slots).tolist()
            hidden = self.r.ws.x[:len(lanes)] if self.has_mtp else None
            self.stats["graph_steps"] = self.stats.get("graph_steps", 0) + 1
        else:
            logits, hidden = self.r.decode(toks, pos, slots)
            new = self._pick_token(logits, [l.req.params for l in lanes], [l.history for l in lanes],
                                   [l.key for l in lanes])
        self.stats["decode_steps"] += 1
        for i, lane in enumerate(lanes):
            self.slot_cache[lane.slot].append(lane.last_tok)          # the FED token; invariant len == pos
            lane.pos += 1
            lane.key = S.splitmix64(lane.key)
            lane.last_tok = new[i]
            lane.generated += 1
            self._push_history(lane, [new[i]])
            # a plain decode leaves the draft head's cache without this position: the lane stops speculating
            lane.mtp_ok = False
            if hidden is not None and self.has_mtp:
                lane.h_prev = hidden[i].clone()
            self._emit(lane, [new[i]])

    # ------------------------------------------------------------------ speculation: drafting
    def _draft_chain(self, lane: Lane, n_drafts: int) -> Tuple[List[int], Optional[torch.Tensor]]:
        """Greedy draft chain from the MTP head: feeds (h, token) pairs, each step reusing the head's own
        hidden. Returns the draft tokens."""
        drafts: List[int] = []
        h = lane.h_prev
        tok = lane.last_tok
        p = lane.pos - 1
        if self.sampler is not None and self.ngram <= 0 and n_drafts > 0 and getattr(self.r, "tp", 1) == 1:
            # the whole chain stays on the device: each step's arg-max feeds the next step's token slot directly and
            # the draft ids come back in one read
            from ..ops import kernels as K
            outs = torch.empty(n_drafts, dtype=torch.int32, device=h.device)
            ids = getattr(self.r, "draft_ids", None)            # draft-vocabulary head: row index -> token id
            tok_dev = None
            for d in range(n_drafts):
                logits, hh = self.r.mtp_forward(lane.slot, [tok if d == 0 else 0], h.reshape(1, -1), [p], tok_dev=tok_dev,
                                                draft_only=True)
                K.argmax(logits, 1, outs[d:d + 1])
                if ids is not None and logits.shape[1] == ids.numel():
                    outs[d:d + 1] = ids[outs[d:d + 1].long()].to(torch.int32)
                tok_dev = outs[d:d + 1]
                h, p = hh[0].clone(), p + 1
            return outs.tolist(), h
        for d in range(n_drafts):
            if self.ngram > 0:
                ng = self._ngram_lookup(lane, drafts)
                if ng is not None and d > 0:
                    drafts.append(ng)
                    # keep the head's cache in step even when its own guess is overridden
                    logits, hh = self.r.mtp_forward(lane.slot, [tok], h.reshape(1, -1), [p])
                    h, tok, p = hh[0].clone(), ng, p + 1
                    continue
            logits, hh = self.r.mtp_forward(lane.slot, [tok], h.reshape(1, -1), [p])
            nxt = self._argmax(logits)[0]
            drafts.append(nxt)
            h, tok, p = hh[0].clone(), nxt, p + 1
        return drafts, h

    def _ngram_lookup(self, lane: Lane, pending: Sequence[int]) -> Optional[int]:
        """Prompt-lookup continuation: the token that followed the last ``ngram`` tokens earlier in the
        sequence (searching from the most recent occurrence)."""
        n = self.ngram
        seq = self.slot_cache[lane.slot] + [lane.last_tok] + list(pending)
        if n <= 0 or len(seq) <= n:
            return None
        key = seq[-n:]
        for s in range(len(seq) - n - 1, -1, -1):
            if seq[s:s + n] == key:
                return seq[s + n]
        return None

    def _reprime(self, lane: Lane, fed: Sequence[int], hidden: torch.Tensor, pos0: int):
        """Rewrite the draft head's cache for the accepted columns with backbone hiddens: pairs
        (hidden[t-1], fed[t]) at head position pos0 - 1 + t for t >= 1."""
        n = len(fed)
        if n > 1:
            self.r.mtp_forward(lane.slot, list(fed[1:]), hidden[:n - 1], [pos0 + t - 1 for t in range(1, n)])

    def _commit(self, lane: Lane, fed: Sequence[int], new_last: int, emitted: Sequence[int], hidden_row: torch.Tensor):
        self.slot_cache[lane.slot].extend(fed)
        lane.pos += len(fed)
        lane.key = S.splitmix64(lane.key)
        lane.last_tok = new_last
        lane.h_prev = hidden_row.clone()
        for t in emitted:
            if lane.done:
                break
            lane.generated += 1
            self._push_history(lane, [t])
            self._emit(lane, [t])

    # ------------------------------------------------------------------ speculation: steps
    def _depth_for(self, lane: Lane, cap: int = MAX_VERIFY_COLS) -> int:
        room = self.max_seq - lane.pos - 1
        return max(1, min(self.policy.depth, cap, room))

    def _verify_chain(self, lane: Lane, cols: Sequence[int]):
        """Chain verify of one lane: a graph replay per width when the runner has one (same kernels, same bits)."""
        if self.use_graphs and hasattr(self.r, "replay_verify") and 1 < len(cols) <= MAX_VERIFY_COLS:
            self.stats["verify_graph_steps"] = self.stats.get("verify_graph_steps", 0) + 1
            return self.r.replay_verify(lane.slot, cols, lane.pos, self.ckpt_base)
        return self.r.verify(lane.slot, cols, lane.pos, self.ckpt_base)

    def _mtp_chain_step(self, lane: Lane):
        depth = self._depth_for(lane)
        drafts, _ = self._draft_chain(lane, depth - 1)
        cols = [lane.last_tok] + drafts
        logits, hidden = self._verify_chain(lane, cols)
        preds = self._greedy_preds(logits, lane, drafts)
        nacc = S.greedy_accept(preds, drafts)
        bonus = preds[nacc]
        pos0 = lane.pos
        self.r.copy_state(self.ckpt_base + nacc, lane.slot)           # recurrent state after column nacc
        fed = cols[:nacc + 1]
        hid = hidden[:nacc + 1].clone()
        self._reprime(lane, fed, hid, pos0)
        self._commit(lane, fed, bonus, drafts[:nacc] + [bonus], hid[nacc])
        self.policy.record_step(len(drafts), nacc, nacc + 1)
        self.stats["mtp_steps"] += 1
        self._log_mtp_step(lane, pos0, cols[0], drafts, preds, nacc)

    def _argmax(self, logits: torch.Tensor) -> List[int]:
        """Greedy token per row (lowest index on ties), over the whole vocabulary even when ``logits`` is one rank's shard."""
        if self.sampler is not None and logits.is_cuda:
            n = logits.shape[0]
            return self.sampler.pick(logits if logits.dtype == torch.float32 else logits.float(),
                                     [SamplingParams(0.0, 1.0, 1)] * n, [[]] * n, [0] * n)
        return S.argmax_rows(logits if logits.dtype == torch.float32 else logits.float())

    def _greedy_preds(self, logits: torch.Tensor, lane: Lane, drafts: Sequence[int]) -> List[int]:
        """Arg-max per verify column; column t is penalised with the history extended by the first t drafts."""
        n = logits.shape[0]
        if self.sampler is not None and logits.is_cuda:
            hists, hist = [], list(lane.history)
            for t in range(n):
                hists.append(list(hist))
                if t < len(drafts):
                    hist.append(drafts[t])
            greedy = SamplingParams(0.0, 1.0, 1, lane.req.params.repetition_penalty, lane.req.params.presence_penalty,
                                    lane.req.params.frequency_penalty)
            return self.sampler.pick(logits if logits.dtype == torch.float32 else logits.float(), [greedy] * n, hists, [0] * n)
        if lane.req.params.has_penalty:
            logits = logits.clone()
            hist = list(lane.history)
            for t in range(n):
                logits[t] = S.apply_penalties(logits[t], hist, lane.req.params)
                if t < len(drafts):
                    hist.append(drafts[t])
        return S.argmax_rows(logits if logits.dtype == torch.float32 else logits.float())

    def _mtp_sample_step(self, lane: Lane):
        depth = self._depth_for(lane)
        drafts, _ = self._draft_chain(lane, depth - 1)
        cols = [lane.last_tok] + drafts
        logits, hidden = self._verify_chain(lane, cols)
        if self.sampler is not None and logits.is_cuda:
            # accept / residual resample / bonus on the device: one read of (accepted, next token) comes back
            nacc, nxt = self.sampler.chain_accept(logits if logits.dtype == torch.float32 else logits.float(),
                                                  lane.req.params, lane.history, drafts, lane.key)
        else:
            logits = logits.clone() if logits.dtype == torch.float32 else logits.float()
            if lane.req.params.has_penalty:
                hist = list(lane.history)
                for t in range(len(cols)):
                    logits[t] = S.apply_penalties(logits[t], hist, lane.req.params)
                    if t < len(drafts):
                        hist.append(drafts[t])
            nuclei = S.nucleus_rows(logits, [lane.req.params] * len(cols))
            nacc, nxt = S.stochastic_accept(nuclei, drafts, lane.key)
        pos0 = lane.pos
        self.r.copy_state(self.ckpt_base + nacc, lane.slot)
        fed = cols[:nacc + 1]
        hid = hidden[:nacc + 1].clone()
        self._reprime(lane, fed, hid, pos0)
        self._commit(lane, fed, nxt, drafts[:nacc] + [nxt], hid[nacc])
        self.policy.record_step(len(drafts), nacc, nacc + 1)
        self.stats["mtp_steps"] += 1
        self._log_mtp_step(lane, pos0, cols[0], drafts, [], nacc)

    def _mtp_tree_step(self, lane: Lane):
        """Fork drafting: branch A is the head's greedy chain, branch B a pure n-gram continuation; the fork
        is kept only when B exists and starts with a different token."""
        depth = self._depth_for(lane)
        ng = self.ngram
        self.ngram = 0
        a, _ = self._draft_chain(lane, depth - 1)
        self.ngram = ng
        b: List[int] = []
        for _ in range(min(depth - 1, MAX_VERIFY_COLS - 1 - len(a))):
            t = self._ngram_lookup(lane, b)
            if t is None:
                break
            b.append(t)
        if not b or not a or b[0] == a[0]:
            b = []
        tokens = [lane.last_tok] + a + b
        parent = [-1] + [i for i in range(len(a))] + ([0] + [len(a) + 1 + i for i in range(len(b) - 1)] if b else [])
        if not b:
            logits, hidden = self.r.verify(lane.slot, tokens, lane.pos, self.ckpt_base)
        else:
            logits, hidden = self.r.verify(lane.slot, tokens, lane.pos, self.ckpt_base, parent=parent)
        preds = self._argmax(logits)
        path = S.tree_accept_walk(parent, tokens, preds)
        nacc = len(path) - 1
        last_col = path[-1]
        bonus = preds[last_col]
        pos0 = lane.pos
        if b and path != list(range(len(path))):
            self.r.compact_kv(lane.slot, pos0, path)
        self.r.copy_state(self.ckpt_base + last_col, lane.slot)
        fed = [tokens[c] for c in path]
        hid = torch.stack([hidden[c] for c in path])
        self._reprime(lane, fed, hid, pos0)
        self._commit(lane, fed, bonus, fed[1:] + [bonus], hid[-1])
        self.policy.record_step(len(a), nacc, nacc + 1)
        self.stats["mtp_steps"] += 1
        self.stats["tree_steps"] += 1

    def _mtp_forest_step(self, lanes: List[Lane]):
        """Pack several greedy lanes' draft chains into one verify of at most 16 columns."""
        p = len(lanes)
        d = max(1, min(self.policy.depth, MAX_VERIFY_COLS // p - 1))
        plans = []
        base = self.ckpt_base
        for lane in lanes:
            depth = max(1, min(d + 1, self.max_seq - lane.pos - 1))
            drafts, _ = self._draft_chain(lane, depth - 1)
            cols = [lane.last_tok] + drafts
            plans.append((lane, cols, drafts, base))
            base += len(cols)
        outs = self.r.verify_forest([(lane.slot, cols, lane.pos, b) for lane, cols, _, b in plans])
        for (lane, cols, drafts, b), (logits, hidden) in zip(plans, outs):
            preds = self._argmax(logits)
            nacc = S.greedy_accept(preds, drafts)
            pos0 = lane.pos
            self.r.copy_state(b + nacc, lane.slot)
            fed = cols[:nacc + 1]
            hid = hidden[:nacc + 1].clone()
            self._reprime(lane, fed, hid, pos0)
            self._commit(lane, fed, preds[nacc], drafts[:nacc] + [preds[nacc]], hid[nacc])
            self.policy.record_step(len(drafts), nacc, nacc + 1)
        self.stats["mtp_steps"] += 1
        self.stats["forest_steps"] += 1

    # ------------------------------------------------------------------ divergence guard
    def state_hash(self) -> int:
        """FNV hash of the lane table; tensor-parallel ranks compare it every step."""
        h = 0xCBF29CE484222325
        for lane in self.lanes:
            for v in (lane.slot, lane.pos, lane.last_tok, lane.generated, lane.req.id):
                h = ((h ^ (v & 0xFFFFFFFF)) * 0x100000001B3) & S.MASK64
        h = ((h ^ self.policy.depth) * 0x100000001B3) & S.MASK64
        return h
