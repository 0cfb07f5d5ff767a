"""Worker for test_lockstep: two CPU (gloo) ranks run oracle-backed schedulers in lockstep."""
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
    try:
        if rank == 0:
            reqs = []
            for i, p in enumerate(([3, 4, 5, 6, 7], [9, 8, 7], [1, 2, 3, 4])):
                sink = []
                r = Request(p, 5, SamplingParams(temperature=0.0), on_token=sink.append)
                reqs.append(r)
                outs[i] = sink
            ls.head_step(reqs[:2], [])
            ls.head_step([], [])
            reqs[1].cancelled = True
            ls.head_step([reqs[2]], [reqs[1].id])
            while not sch.idle():
                ls.head_step([], [])
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
