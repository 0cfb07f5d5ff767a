"""Worker for test_gpu_comm: a tensor-parallel tiny model must agree with the single-GPU model (to rounding),
be deterministic run to run, and keep verify == sequential decode at this world size."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from velogb10_b200.checkpoint.synthetic import SyntheticSource
    from velogb10_b200.config import tiny_hybrid
    from velogb10_b200.models.runtime import GpuModel
    from velogb10_b200.models.weights import ModelBuilder
    from velogb10_b200.parallel.comm import TpComm
    cfg = tiny_hybrid(mtp=False)
    cfg.num_heads, cfg.num_kv_heads = 4, 2
    comm = TpComm(rank, world, dev, max_elems=1 << 20)
    w1 = ModelBuilder(cfg, SyntheticSource(cfg, 0, str(dev), std=0.05), recipe="all", device=str(dev)).build()
    wt = ModelBuilder(cfg, SyntheticSource(cfg, 0, str(dev), std=0.05), recipe="all", device=str(dev), tp_rank=rank,
                      tp_world=world).build()
    single = GpuModel(w1, device=str(dev))
    tp = GpuModel(wt, device=str(dev), comm=comm)
    single.alloc_state(2, 2 + 17, 512)
    tp.alloc_state(2, 2 + 17, 512)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, cfg.vocab_size, (300,), generator=g).tolist()
    l1, _ = single.prefill(0, prompt)
    lt, _ = tp.prefill(0, prompt)
    torch.cuda.synchronize()
    comm.check()
    rel = ((lt.float() - l1.float()).norm() / l1.float().norm()).item()
    assert lt.shape == l1.shape and rel < 0.05, rel
    # prefill widths run the GEMM fused with the reduce-scatter; the unfused form (GEMM, then two-shot all-reduce)
    # must agree to rounding, and the fused form must be deterministic
    tp.fuse_allreduce = False
    lu0, _ = tp.prefill(1, prompt)
    tp.fuse_allreduce = True
    tp.zero_slot(1)
    lf0, _ = tp.prefill(1, prompt)
    torch.cuda.synchronize()
    comm.check()
    assert torch.equal(lf0, lt)
    relu = ((lu0.float() - lt.float()).norm() / lt.float().norm()).item()
    assert relu < 0.02, relu
    # verify == sequential decodes at this world size, and run-to-run determinism
    S0, C0, K0, V0 = tp.S.clone(), tp.conv.clone(), tp.kc.clone(), tp.vc.clone()
    toks = [int(lt.argmax()), 5, 7, 11]
    lv, _ = tp.verify(0, toks, 300, ckpt_base=2)
    lv = lv.clone()
    tp.S.copy_(S0); tp.conv.copy_(C0); tp.kc.copy_(K0); tp.vc.copy_(V0)
    lv2, _ = tp.verify(0, toks, 300, ckpt_base=2)
    assert torch.equal(lv, lv2)
    tp.S.copy_(S0); tp.conv.copy_(C0); tp.kc.copy_(K0); tp.vc.copy_(V0)
    for t in range(4):
        ld, _ = tp.decode([toks[t]], [300 + t], [0])
        assert torch.equal(ld[0], lv[t]), t
    # the fused GEMM-epilogue all-reduce and the separate all-reduce kernel give the same tokens
    tp.S.copy_(S0); tp.conv.copy_(C0); tp.kc.copy_(K0); tp.vc.copy_(V0)
    tp.fuse_allreduce = False
    lu, _ = tp.verify(0, toks, 300, ckpt_base=2)
    tp.fuse_allreduce = True
    rel = ((lu.float() - lv.float()).norm() / lv.float().norm()).item()
    assert rel < 0.02 and lu.argmax(-1).tolist() == lv.argmax(-1).tolist(), rel
    # graph replay under tensor parallelism
    tp.S.copy_(S0); tp.conv.copy_(C0); tp.kc.copy_(K0); tp.vc.copy_(V0)
    want = int(lv[0].argmax())
    got = int(tp.replay_decode([toks[0]], [300], [0])[0])
    assert got == want, (got, want)
    torch.cuda.synchronize()
    comm.check()
    dist.barrier()
    if rank == 0:
        print("TP_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
