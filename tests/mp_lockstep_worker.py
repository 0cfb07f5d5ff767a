"""Worker for test_lockstep: two CPU (gloo) ranks run oracle-backed schedulers in lockstep.

LOCKSTEP_MODE selects the scenario: (default) replay + cancellation, including a cancel flag that flips between the
head's snapshot and the step and a cancelled request that is still queued; ``leave``: rank 1 exits between steps
without answering; ``fault``: rank 1's health probe reports a kernel failure at its third step."""
import os
import sys

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    from velogb10_b200.checkpoint.synthetic import SyntheticSource
    from velogb10_b200.config import tiny_hybrid
    from velogb10_b200.engine.mtp import MtpPolicy
    from velogb10_b200.engine.sampling import SamplingParams
    from velogb10_b200.engine.scheduler import Request, Scheduler
    from velogb10_b200.models.oracle import OracleModel
    from velogb10_b200.models.weights import ModelBuilder
    from velogb10_b200.parallel.lockstep import DivergenceError, Lockstep, make_cpu_group
    cfg = tiny_hybrid(mtp=False)
    w = ModelBuilder(cfg, SyntheticSource(cfg, 0, std=0.08), recipe="all").build()
    sch = Scheduler(OracleModel(w), 2, 96, eos_ids=[], policy=MtpPolicy("off"))
    ls = Lockstep(sch, make_cpu_group(5.0))
    outs = {}
    mode = os.environ.get("LOCKSTEP_MODE", "")
    if mode == "fault" and rank == 1:
        from velogb10_b200.ops.lib import KernelError
        calls = [0]

        def probe():
            calls[0] += 1
            if calls[0] == 3:
                raise KernelError("a kernel reported bounded-wait failure code 4")
        sch.health_check = probe
    try:
        if mode in ("leave", "fault"):
            if rank == 0:
                ls.head_step([Request([3, 4, 5, 6, 7], 40, SamplingParams(temperature=0.0))], [])
                for _ in range(8):
                    ls.head_step([], [])
                ls.head_step([], [], stop=True)
            else:
                steps = 0
                while ls.mirror_step():
                    steps += 1
                    if mode == "leave" and steps == 2:
                        # between steps: nothing of this rank is in flight; it simply never answers again
                        os._exit(0)
            print(f"UNEXPECTED_END rank {rank}")
            sys.exit(0)
        if rank == 0:
            reqs = []
            for i, p in enumerate(([3, 4, 5, 6, 7], [9, 8, 7], [1, 2, 3, 4])):
                sink = []
                r = Request(p, 5, SamplingParams(temperature=0.0), on_token=sink.append)
                reqs.append(r)
                outs[i] = sink
            fin = {}
            for i, r in enumerate(reqs):
                r.on_finish = (lambda i_: lambda reason, u: fin.__setitem__(i_, reason))(i)
            late = Request([5, 5, 5], 30, SamplingParams(temperature=0.0), on_finish=lambda reason, u: fin.__setitem__("late", reason))
            queued = Request([6, 6, 6], 5, SamplingParams(temperature=0.0), on_finish=lambda reason, u: fin.__setitem__("queued", reason))
            ls.head_step(reqs[:2], [])
            ls.head_step([], [])
            reqs[1].cancelled = True
            ls.head_step([reqs[2]], sch.pending_cancels())
            assert fin.get(1) == "cancelled", fin          # a cancelled lane still gets its final event
            while not sch.idle():
                ls.head_step([], sch.pending_cancels())
            # the flag flips after the head took its snapshot: this step must not act on it (the mirrors cannot know)
            ls.head_step([late, queued, Request([7, 7], 30, SamplingParams(temperature=0.0))], [])
            snap = sch.pending_cancels()
            late.cancelled = True
            queued.cancelled = True                          # still waiting for a slot (two lanes are busy)
            n_before = len(sch.lanes)
            ls.head_step([], snap)
            assert len(sch.lanes) == n_before and "late" not in fin, (fin, len(sch.lanes))
            ls.head_step([], sch.pending_cancels())
            assert fin.get("late") == "cancelled", fin
            for r_ in [l.req for l in sch.lanes]:
                r_.cancelled = True
            while not sch.idle():
                ls.head_step([], sch.pending_cancels())
            assert fin.get("queued") == "cancelled", fin
            ls.head_step([], [], stop=True)
            toks = [outs[0], outs[2]]
        else:
            while ls.mirror_step():
                pass
            toks = [ls.mirror_reqs[1][1], ls.mirror_reqs[3][1]]
        allt = [None, None]
        dist.all_gather_object(allt, toks)
        assert allt[0] == allt[1] and len(allt[0][0]) == 5, allt
        print(f"LOCKSTEP_OK rank {rank}")
    except DivergenceError as e:
        print(f"DIVERGED rank {rank}: {e}")
        sys.exit(3)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
