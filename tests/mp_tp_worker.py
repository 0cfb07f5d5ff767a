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
    # enough heads to shard at this world size (KV heads are replicated when there are fewer of them than ranks)
    cfg.num_heads, cfg.num_kv_heads = max(4, world), 2
    cfg.lin_num_k_heads, cfg.lin_num_v_heads = max(4, world), 2 * max(4, world)
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
    # every rank holds the same residual stream, bit for bit (the sums are order-fixed or made once in the switch)
    hid = comm.all_gather_small(tp.ws.x[:1].contiguous().view(torch.int16))
    torch.cuda.synchronize()
    assert all(torch.equal(hid[0], hid[q]) for q in range(world)), "ranks diverged in the residual stream"
    # graph replay under tensor parallelism
    tp.S.copy_(S0); tp.conv.copy_(C0); tp.kc.copy_(K0); tp.vc.copy_(V0)
    want = int(lv[0].argmax())
    got = int(tp.replay_decode([toks[0]], [300], [0])[0])
    assert got == want, (got, want)
    torch.cuda.synchronize()
    comm.check()
    # mixture-of-experts under tensor + expert parallelism (expert bands, forked shared expert, grouped FP4 GEMMs)
    from velogb10_b200.config import tiny_moe
    from velogb10_b200.ops import gemm as G
    mcfg = tiny_moe(mtp=False)
    mcfg.num_heads, mcfg.lin_num_k_heads, mcfg.lin_num_v_heads = max(4, world), max(4, world), 2 * max(4, world)
    m1 = GpuModel(ModelBuilder(mcfg, SyntheticSource(mcfg, 0, str(dev), std=0.05), recipe="all", device=str(dev)).build(),
                  device=str(dev))
    mt = GpuModel(ModelBuilder(mcfg, SyntheticSource(mcfg, 0, str(dev), std=0.05), recipe="all", device=str(dev),
                               tp_rank=rank, tp_world=world).build(), device=str(dev), comm=comm)
    m1.alloc_state(2, 2 + 17, 256)
    mt.alloc_state(2, 2 + 17, 256)
    # end to end with the single-GPU run's router logits replayed on the tensor-parallel model: both then route every
    # token identically, and what remains is the summation order of the expert-parallel reduction and of the sharded
    # mixers, so the logits must agree to the tolerance of the dense tensor-parallel model
    mp = torch.randint(0, mcfg.vocab_size, (90,), generator=g).tolist()
    rec = []
    m1.router_logits_hook = lambda lg, n_: rec.append(lg[:n_].clone())
    a1, _ = m1.prefill(0, mp)
    d1, _ = m1.decode([5, 7], [90, 3], [0, 1])
    d1 = d1.clone()
    m1.router_logits_hook = None
    it = iter(rec)
    mt.router_logits_hook = lambda lg, n_: lg[:n_].copy_(next(it))
    at, _ = mt.prefill(0, mp)
    dt, _ = mt.decode([5, 7], [90, 3], [0, 1])
    mt.router_logits_hook = None
    dt2 = dt.clone()
    torch.cuda.synchronize()
    comm.check()
    rel_p = ((at.float() - a1.float()).norm() / a1.float().norm()).item()
    rel_d = ((dt.float() - d1.float()).norm() / d1.float().norm()).item()
    print("moe prefill rel", rel_p, "decode rel", rel_d, flush=True)
    assert rel_p < 0.06 and rel_d < 0.06, ("moe end to end with replayed routing", rel_p, rel_d)
    # layer level, identical inputs on both models (so the routing is identical and only the summation order of
    # the expert-parallel reduction differs): per-pair decode path and sorted prefill path
    for ws1, wst, n in ((m1.ws, mt.ws, 2), (m1.ws_prefill, mt.ws_prefill, 90)):
        xin = (torch.randn((n, mcfg.hidden_size), generator=g) * 0.5).to(dev, torch.float16)
        outs = []
        for m, ws in ((m1, ws1), (mt, wst)):
            ws.xn16[:n].copy_(xin)
            moe = next(L.moe for L in m.w.layers if L.moe is not None)
            act = G.quantize_act_fp4(ws.xn16, n, ((mcfg.hidden_size + 255) // 256) * 256) if (m.use_fp4 and n <= 16) else None
            ws.x[:n].zero_()
            m._moe(ws, moe, n, act=act)
            if m._pending_ar:
                # the combine only pushed this rank's partial rows: the residual-add / RMSNorm kernel sums the ranks
                m._norm(ws, None, m.w.final_norm, n)
                outs.append(ws.x[:n].float().clone())
            else:
                outs.append(ws.delta[:n].float().clone())
        rel = ((outs[1] - outs[0]).norm() / outs[0].norm()).item()
        assert rel < 0.02, ("moe layer", n, rel)
    torch.cuda.synchronize()
    comm.check()
    # failure detection on the serving path: after a peer wait ran out (a flag nothing sets, 50 ms budget), the
    # scheduler's per-step health probe must raise within two steps, on every rank
    from velogb10_b200.engine.mtp import MtpPolicy
    from velogb10_b200.engine.sampling import SamplingParams
    from velogb10_b200.engine.scheduler import Request, Scheduler
    from velogb10_b200.parallel.comm import CommError
    sch = Scheduler(tp, 2, 256, eos_ids=[], policy=MtpPolicy("off"))
    sch.submit(Request(prompt[:20], 12, SamplingParams(temperature=0.0)))
    sch.step()
    sch.step()
    dist.barrier()
    comm.wait_timeout_probe(0.05)
    raised = False
    try:
        for _ in range(3):
            sch.step()
    except CommError:
        raised = True
    assert raised, "the scheduler kept stepping after a collective reported a timeout"
    torch.cuda.synchronize()
    dist.barrier()
    both = comm.all_gather_small(dt2[:1, :64].contiguous())
    torch.cuda.synchronize()
    assert torch.equal(both[0], both[-1]), "ranks must hold identical logits"
    dist.barrier()
    if rank == 0:
        print("TP_DESC", comm.describe())
        print("TP_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except BaseException:
        import traceback
        print(f"WORKER_FAILED rank {os.environ.get('RANK')}\n" + traceback.format_exc()[-1500:], flush=True)
        raise
