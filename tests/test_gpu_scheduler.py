"""The serving scheduler on the CUDA runtime: greedy output is identical however the work is batched or
speculated (continuous batching, CUDA-graph decode, MTP chain / tree verification, prefix cache)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def weights():
    from velogb10_b200.checkpoint.synthetic import SyntheticSource
    from velogb10_b200.config import tiny_hybrid
    from velogb10_b200.models.weights import ModelBuilder
    cfg = tiny_hybrid(mtp=True)
    return ModelBuilder(cfg, SyntheticSource(cfg, 0, "cuda", std=0.08), recipe="all", device="cuda").build()


def _prompts(cfg, n, seed=1, lo=8, hi=40):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab_size - 2, (int(torch.randint(lo, hi, (1,), generator=g)),), generator=g).tolist()
            for _ in range(n)]


def _run(model, prompts, max_new=14, max_batch=4, policy=None, **kw):
    from velogb10_b200.engine.mtp import MtpPolicy
    from velogb10_b200.engine.sampling import SamplingParams
    from velogb10_b200.engine.scheduler import Request, Scheduler
    sch = Scheduler(model, max_batch, 160, eos_ids=[model.cfg.vocab_size - 1],
                    policy=policy or MtpPolicy("off", has_head=True), **kw)
    outs = [[] for _ in prompts]
    for i, p in enumerate(prompts):
        sch.submit(Request(p, max_new, SamplingParams(temperature=0.0), on_token=outs[i].append))
    sch.run_until_idle(10000)
    torch.cuda.synchronize()
    from velogb10_b200.ops import lib
    lib.check_err_word()
    return outs, sch


def test_batching_speculation_and_prefix_cache_do_not_change_greedy_output(weights):
    from velogb10_b200.engine.mtp import MtpPolicy
    from velogb10_b200.models.runtime import GpuModel
    gm = GpuModel(weights, keep_canonical=True)
    prompts = _prompts(weights.cfg, 5)
    solo = [_run(gm, [p], max_batch=1)[0][0] for p in prompts]
    together, sch = _run(gm, prompts, max_batch=4)
    assert together == solo
    assert sch.stats["admitted"] == 5 and not sch.lanes
    # the model has a draft head and the decode steps still ran as CUDA-graph replays
    assert sch.has_mtp and sch.stats.get("graph_steps", 0) > 0 and sch.stats["graph_steps"] == sch.stats["decode_steps"]
    # bitwise-lossless speculation: the draft head proposes, a width-N verify decides
    for depth in (2, 4):
        spec, sch = _run(gm, prompts[:2], max_batch=1, policy=MtpPolicy("on", depth=depth))
        assert spec == solo[:2], depth
        # the verifies ran as graph replays of that width, and without graphs the text is the same
        assert sch.stats.get("verify_graph_steps", 0) == sch.stats["mtp_steps"] > 0
        eager, sch_e = _run(gm, prompts[:2], max_batch=1, policy=MtpPolicy("on", depth=depth), use_graphs=False)
        assert eager == solo[:2] and sch_e.stats.get("verify_graph_steps", 0) == 0
    # several greedy lanes speculate together: their chains are packed into one forest verify (a graph per shape)
    forest, sch_f = _run(gm, prompts, max_batch=4, policy=MtpPolicy("on", depth=3), mtp_lanes=True)
    assert forest == solo and sch_f.stats["forest_steps"] > 0
    assert any(k[0] == "forest" for k in gm.graphs)
    tree, _ = _run(gm, prompts[:2], max_batch=1, policy=MtpPolicy("on", depth=3), tree_draft=True)
    assert tree == solo[:2]
    # a prompt that extends a served one re-uses the slot's state
    again, sch = _run(gm, [prompts[0], prompts[0] + solo[0][:4]], max_batch=1)
    assert again[0] == solo[0] and again[1] == solo[0][4:] + again[1][len(solo[0]) - 4:]


def test_four_bit_cache_serving_is_self_consistent(weights, monkeypatch):
    from velogb10_b200.engine.mtp import MtpPolicy
    from velogb10_b200.models.runtime import GpuModel
    monkeypatch.setenv("VELO_KV_QUANT", "q4")
    gm = GpuModel(weights, keep_canonical=True)
    prompts = _prompts(weights.cfg, 3, seed=5)
    solo = [_run(gm, [p], max_batch=1)[0][0] for p in prompts]
    together, _ = _run(gm, prompts, max_batch=4)
    spec, _ = _run(gm, prompts[:2], max_batch=1, policy=MtpPolicy("on", depth=3))
    assert together == solo and spec == solo[:2]


def _run_sampling(model, prompts, params, max_new=12, max_batch=4, policy=None, monkeypatch=None, cpu=False):
    from velogb10_b200.engine.mtp import MtpPolicy
    from velogb10_b200.engine.scheduler import Request, Scheduler
    if monkeypatch is not None:
        monkeypatch.setenv("VELO_CPU_SAMPLE", "1" if cpu else "0")
    sch = Scheduler(model, max_batch, 160, eos_ids=[model.cfg.vocab_size - 1], policy=policy or MtpPolicy("off", has_head=True))
    outs = [[] for _ in prompts]
    for i, p in enumerate(prompts):
        sch.submit(Request(p, max_new, params[i], on_token=outs[i].append))
    sch.run_until_idle(10000)
    torch.cuda.synchronize()
    model.gather_logits = True
    return outs, sch


def test_device_sampling_graph_and_speculative_accept(weights, monkeypatch):
    """Seeded sampling and penalised greedy run through the decode + sample graph on the device; the same seeds give
    the same text again; penalised greedy equals the host path exactly; stochastic speculation runs its accept rule
    on the device and stays seed-reproducible."""
    from velogb10_b200.engine.mtp import MtpPolicy
    from velogb10_b200.engine.sampling import SamplingParams
    from velogb10_b200.models.runtime import GpuModel
    gm = GpuModel(weights, keep_canonical=True)
    prompts = _prompts(weights.cfg, 4, seed=9)
    samp = [SamplingParams(0.8, 0.9, 20, seed=100 + i) for i in range(4)]
    a, sch = _run_sampling(gm, prompts, samp, monkeypatch=monkeypatch)
    assert sch.sampler is not None and sch.stats.get("graph_steps", 0) == sch.stats["decode_steps"] > 0
    b, _ = _run_sampling(gm, prompts, samp, monkeypatch=monkeypatch)
    assert a == b and all(len(x) >= 1 for x in a)
    pen = [SamplingParams(0.0, 0.8, 20, 1.3, 0.7, 0.2) for _ in range(4)]
    dev_out, _ = _run_sampling(gm, prompts, pen, monkeypatch=monkeypatch)
    host_out, sch_h = _run_sampling(gm, prompts, pen, monkeypatch=monkeypatch, cpu=True)
    assert sch_h.sampler is None and dev_out == host_out
    # penalised greedy under speculation is still lossless (the verify columns are penalised with the growing history)
    spec_out, _ = _run_sampling(gm, prompts[:2], pen[:2], max_batch=1, policy=MtpPolicy("on", depth=3), monkeypatch=monkeypatch)
    solo_out = [_run_sampling(gm, [p], [pen[0]], max_batch=1, monkeypatch=monkeypatch)[0][0] for p in prompts[:2]]
    assert spec_out == solo_out
    s1, sch1 = _run_sampling(gm, prompts[:2], samp[:2], max_batch=1, policy=MtpPolicy("on", depth=3), monkeypatch=monkeypatch)
    s2, _ = _run_sampling(gm, prompts[:2], samp[:2], max_batch=1, policy=MtpPolicy("on", depth=3), monkeypatch=monkeypatch)
    assert s1 == s2 and sch1.stats["mtp_steps"] > 0 and all(len(x) >= 1 for x in s1)
    from velogb10_b200.ops import lib
    lib.check_err_word()
