"""Lockstep scheduling for multi-process tensor parallelism.

Every rank runs the same scheduler over its shard of the model; rank 0 (the head) owns the HTTP server and
decides what is admitted or cancelled. Before acting on a step the head ships that step's events to the
mirrors, which replay them with dummy callbacks, so all ranks launch the same kernels in the same order.
After every step the ranks compare a hash of their lane tables over a CPU (gloo) group; a mismatch or a
timeout raises ``DivergenceError`` on every rank and the process exits (recovery is a restart, never a
partial repair). This is the counterpart of the reference's head / mirror schedulers and per-step agree
(reference: src/batch.rs:773-942, src/tp_serve.rs:26-116, native/net_shim.c:685-707) on a CPU side channel
instead of the RDMA queue pair.

``VELO_TP_AGREE_DRILL=N`` corrupts this rank's hash at step N (fault-injection drill: the guard must trip).
"""
from __future__ import annotations

import datetime
import os
from dataclasses import asdict
from typing import List, Optional

import torch.distributed as dist

from ..engine.sampling import SamplingParams
from ..engine.scheduler import Request, Scheduler


class DivergenceError(RuntimeError):
    pass


def make_cpu_group(timeout_s: float = 10.0):
    """A gloo group over all ranks for control messages (works whatever the default backend is)."""
    return dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))


def wire_request(req: Request) -> dict:
    return {"id": req.id, "prompt": list(req.prompt), "max_new_tokens": req.max_new_tokens,
            "params": asdict(req.params), "stop_ids": sorted(req.stop_ids), "ckpt_at": req.ckpt_at}


def unwire_request(d: dict, sink: Optional[list] = None) -> Request:
    r = Request(d["prompt"], d["max_new_tokens"], SamplingParams(**d["params"]), set(d["stop_ids"]), d["ckpt_at"])
    if sink is not None:
        r.on_token = sink.append
    return r


class Lockstep:
    def __init__(self, sched: Scheduler, group=None, rank: Optional[int] = None):
        self.s = sched
        self.group = group if group is not None else make_cpu_group()
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size()
        self.step_no = 0
        self.drill = int(os.environ.get("VELO_TP_AGREE_DRILL", "-1"))
        self.mirror_reqs = {}
        # every rank cancels exactly the ids the head broadcast for the step, never from a live flag
        sched.external_cancels = True

    # ---- head side
    def head_step(self, admits: List[Request], cancels: List[int], stop: bool = False):
        """Ship this step's events, then apply them locally and run one scheduler step."""
        for r in admits:
            self.s.submit(r)            # queues the request and assigns its id; nothing runs before the step
        msg = [{"admits": [wire_request(r) for r in admits], "cancels": list(cancels), "stop": stop}]
        self._broadcast(msg)
        if stop:
            return
        self.s.apply_cancels(set(cancels))
        self.agree(self._guarded_step())

    # ---- mirror side
    def mirror_step(self) -> bool:
        msg = [None]
        self._broadcast(msg)
        ev = msg[0]
        if ev["stop"]:
            return False
        for d in ev["admits"]:
            sink: list = []
            r = unwire_request(d, sink)
            self.s.submit(r)
            self.mirror_reqs[d["id"]] = (r, sink)
        self.s.apply_cancels(set(ev["cancels"]))
        self.agree(self._guarded_step())
        return True

    # ---- both
    def _broadcast(self, msg: list):
        try:
            dist.broadcast_object_list(msg, src=0, group=self.group)
        except Exception as e:  # noqa: BLE001 - a peer that closed its connection or timed out ends the run
            raise DivergenceError(f"step {self.step_no}: the step's events could not be exchanged ({e})") from e

    def _guarded_step(self) -> Optional[str]:
        """One scheduler step; a kernel or collective failure reported by the runner's health probe (a bounded
        wait that ran out, a peer's flag that never came) is returned as text instead of raised, so this rank
        still reaches ``agree`` and every rank leaves together."""
        from ..ops.lib import KernelError
        from .comm import CommError
        try:
            self.s.step()
        except (KernelError, CommError) as e:
            return f"rank {self.rank}: {e}"
        return None

    def agree(self, fault: Optional[str] = None):
        h = self.s.state_hash()
        if self.step_no == self.drill and self.rank == self.world - 1:
            h ^= 0xDEAD
        mine = (self.step_no, len(self.s.lanes), h, fault)
        allv = [None] * self.world
        try:
            dist.all_gather_object(allv, mine, group=self.group)
        except Exception as e:  # noqa: BLE001 - a silent or dead peer ends the run
            raise DivergenceError(f"step {self.step_no}: a rank did not answer ({e})") from e
        self.step_no += 1
        faults = [v[3] for v in allv if v[3]]
        if faults:
            raise DivergenceError(f"step {mine[0]}: device failure reported: {'; '.join(faults)}")
        if any(v[:3] != allv[0][:3] for v in allv):
            raise DivergenceError(f"ranks diverged at step {mine[0]}: {allv}")


def run_mirror(sched: Scheduler, group=None):
    ls = Lockstep(sched, group)
    while ls.mirror_step():
        pass
