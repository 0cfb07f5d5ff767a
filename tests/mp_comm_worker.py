"""Worker for test_gpu_comm: checks the peer-memory all-reduce / all-gather / arg-max merge against the
library collectives, determinism across repeats and graph replay, and the bounded-wait error path."""
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
    from velogb10_b200.parallel.comm import CommError, TpComm
    comm = TpComm(rank, world, dev, max_elems=1 << 22, timeout_s=5.0, ag_bytes=2 * 256 * world * 1024 * 2)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    for rows, h in ((1, 5120), (16, 5120), (3, 256), (700, 5120)):      # one-shot and two-shot sizes
        x = torch.randn(rows, h, generator=g, device=dev).to(torch.bfloat16)
        ref = x.float().clone()
        dist.all_reduce(ref)
        for rep in range(3):
            y = x.clone()
            comm.all_reduce_rows(y, rows)
            torch.cuda.synchronize()
            comm.check()
            err = (y.float() - ref).abs().max().item()
            assert err <= 0.02 * ref.abs().max().item() + 1e-3, (rows, h, rep, err)
            if rep == 0:
                first = y.clone()
            assert torch.equal(y, first), "all-reduce must be deterministic"
        # every rank holds identical bits
        both = comm.all_gather_small(first[:1, :64].contiguous())
        torch.cuda.synchronize()
        assert torch.equal(both[0], both[-1])
    # in-switch all-reduce (multicast-bound symmetric buffer), in place: close to the fp32 reference, identical on
    # every rank and on every repeat
    sb = comm.symmetric_buffer(700 * 5120 * 2)
    if sb is not None:
        t = sb.view(torch.bfloat16).view(700, 5120)
        x = torch.randn(700, 5120, generator=g, device=dev).to(torch.bfloat16)
        ref = x.float().clone()
        dist.all_reduce(ref)
        for rep in range(3):
            t.copy_(x)
            dist.barrier()                      # no rank may still be reading the previous result
            assert comm.all_reduce_multimem(t, 700)
            torch.cuda.synchronize()
            comm.check()
            err = (t.float() - ref).abs().max().item()
            assert err <= 0.02 * ref.abs().max().item() + 1e-3, ("multimem all-reduce", rep, err)
            if rep == 0:
                first = t.clone()
            assert torch.equal(t, first)
        both = comm.all_gather_small(first[:1, :64].contiguous())
        torch.cuda.synchronize()
        assert all(torch.equal(both[0], both[q]) for q in range(world))
    # graph replay advances the device-side epoch by itself
    x = torch.randn(4, 1024, generator=g, device=dev).to(torch.bfloat16)
    buf = x.clone()
    comm.all_reduce_rows(buf, 4)
    torch.cuda.synchronize()
    want = buf.clone()
    buf.copy_(x)
    gr = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        comm.all_reduce_rows(buf, 4)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    dist.barrier()
    buf.copy_(x)
    with torch.cuda.graph(gr):
        comm.all_reduce_rows(buf, 4)
    for _ in range(3):
        buf.copy_(x)
        gr.replay()
        torch.cuda.synchronize()
        assert torch.equal(buf, want)
    comm.check()
    # vocabulary-parallel arg-max
    logits = torch.randn(5, 1000, generator=g, device=dev)
    toks = comm.argmax_vocab_parallel(logits)
    full = comm.gather_logits(logits)
    assert toks == full.argmax(-1).tolist()
    # bounded wait: a flag nothing sets times out, reports, and leaves the context usable
    dist.barrier()
    comm.wait_timeout_probe(0.05)
    torch.cuda.synchronize()
    try:
        comm.check()
        raise AssertionError("timeout was not reported")
    except CommError:
        pass
    y = x.clone()
    comm.all_reduce_rows(y, 4)
    torch.cuda.synchronize()
    comm.check()
    assert torch.equal(y, want)
    # fused all-gather + GEMM: token rows sharded over the ranks, every rank computes the full product
    from velogb10_b200.models.weights import QLinear
    n_total, K_, M_ = 256 * world - 84, 1024, 384        # every rank's shard is non-empty, the last one ragged
    gw = torch.Generator(device=dev).manual_seed(7)                       # same weights and inputs on every rank
    w = (torch.randn(M_, K_, generator=gw, device=dev) * 0.05).to(torch.bfloat16)
    xf = torch.randn(n_total, K_, generator=gw, device=dev).to(torch.float16)
    q = QLinear.from_dense(w, "nvfp4")
    rows_per = ((n_total + world - 1) // world + 127) // 128 * 128
    r0, r1 = min(n_total, rank * rows_per), min(n_total, (rank + 1) * rows_per)
    ref = (xf.float() @ q.dequant(torch.float32).t())
    for rep in range(3):                                                   # both landing zones, repeated epochs
        shard = (xf[r0:r1] * (rep + 1)).contiguous()
        out = torch.zeros(n_total, M_, dtype=torch.bfloat16, device=dev)
        comm.ag_gemm(q, shard, r0, n_total, out)
        torch.cuda.synchronize()
        comm.check()
        rel = ((out.float() - ref * (rep + 1)).norm() / (ref * (rep + 1)).norm()).item()
        assert rel < 1e-2, (rep, rel)
    # fused decode-width all-reduce: the row-parallel FP4 GEMM's epilogue publishes its partial rows and the
    # residual-add / RMSNorm kernel sums the ranks (in the NVLink switch when the arena is multicast-bound, else
    # from (value, epoch) pairs); same bits on every rank and on every repeat
    from velogb10_b200.ops import gemm as G
    h, kloc = 5120, 1024
    wf = (torch.randn(h, kloc * world, generator=gw, device=dev) * 0.05).to(torch.bfloat16)
    xa = torch.randn(16, kloc * world, generator=gw, device=dev).to(torch.float16)
    qs = [QLinear.from_dense(wf[:, r * kloc:(r + 1) * kloc].contiguous(), "nvfp4") for r in range(world)]
    ref = sum(xa[:, r * kloc:(r + 1) * kloc].float() @ qs[r].dequant(torch.float32).t() for r in range(world))
    x_loc = xa[:, rank * kloc:(rank + 1) * kloc].contiguous()
    ones = torch.zeros(h, device=dev)
    x16 = torch.zeros(16, h, dtype=torch.float16, device=dev)
    dummy = torch.zeros(16, h, dtype=torch.bfloat16, device=dev)
    mode = 2 if comm.use_mm else 1
    for n in (1, 5, 16):
        for rep in range(4):
            res = torch.zeros(16, h, dtype=torch.bfloat16, device=dev)
            G.linear_fp4(qs[rank], x_loc, n, out=dummy, comm=comm, push_only=True)
            G.add_rmsnorm_fp4_ar(res, ones, 1e-6, n, comm, out16=x16, mode=mode)
            torch.cuda.synchronize()
            comm.check()
            rel = ((res[:n].float() - ref[:n]).norm() / ref[:n].norm()).item()
            assert rel < 8e-3, ("fused all-reduce", n, rep, rel)
            if rep == 0:
                first = res.clone()
            assert torch.equal(res, first), "fused all-reduce must be deterministic"
        both = comm.all_gather_small(first[:1, :64].contiguous())
        torch.cuda.synchronize()
        assert torch.equal(both[0], both[-1]), "ranks must hold identical sums"
    # device-side sampling over a vocabulary-sharded head: same token on every rank, equal to the full-logits result
    from velogb10_b200.engine import sampling as S
    from velogb10_b200.engine.device_sampler import DeviceSampler
    vl = 3000
    full_logits = (torch.randn(6, vl * world, generator=gw, device=dev) * 3 * 4).round() / 4
    params = [S.SamplingParams(0.7, 0.8, 20), S.SamplingParams(0.0, 0.8, 20), S.SamplingParams(1.2, 0.95, 64)] * 2
    sh = DeviceSampler(dev, vl, cap=16, comm=comm)
    one = DeviceSampler(dev, vl * world, cap=16)
    keys = [3, 5, 7, 11, 13, 17]
    got = sh.pick(full_logits[:, rank * vl:(rank + 1) * vl].contiguous(), params, [[]] * 6, keys)
    want = one.pick(full_logits.clone(), params, [[]] * 6, keys)
    comm.check()
    assert got == want, (got, want)
    dist.barrier()
    if rank == 0:
        print("COMM_DESC", comm.describe())
        print("COMM_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except BaseException:
        import traceback
        print(f"WORKER_FAILED rank {os.environ.get('RANK')}\n" + traceback.format_exc()[-1500:], flush=True)
        raise
