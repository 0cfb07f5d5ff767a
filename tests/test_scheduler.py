"""Scheduler behaviour on the fp32 CPU oracle: plumbing of slots, prefix cache, speculation variants.
Greedy output must be identical however the work is batched or speculated."""
import pytest
import torch

from velogb10_b200.checkpoint.synthetic import SyntheticSource
from velogb10_b200.config import tiny_hybrid, tiny_moe
from velogb10_b200.engine import sampling as S
from velogb10_b200.engine.mtp import MtpPolicy
from velogb10_b200.engine.sampling import SamplingParams
from velogb10_b200.engine.scheduler import Request, Scheduler
from velogb10_b200.models.oracle import OracleModel
from velogb10_b200.models.weights import ModelBuilder

GREEDY = SamplingParams(temperature=0.0)


@pytest.fixture(scope="module")
def weights():
    cfg = tiny_hybrid(mtp=True)
    return ModelBuilder(cfg, SyntheticSource(cfg, 0, std=0.08), recipe="all").build()


def _prompts(cfg, n, seed=1, lo=8, hi=40):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab_size - 2, (int(torch.randint(lo, hi, (1,), generator=g)),), generator=g).tolist()
            for _ in range(n)]


def _run(weights, prompts, max_new=12, params=GREEDY, max_batch=4, policy=None, **kw):
    orc = OracleModel(weights)
    sch = Scheduler(orc, max_batch, 128, eos_ids=[weights.cfg.vocab_size - 1],
                    policy=policy or MtpPolicy("off", has_head=True), **kw)
    outs = [[] for _ in prompts]
    fins = [None] * len(prompts)
    for i, p in enumerate(prompts):
        sch.submit(Request(p, max_new, params, on_token=outs[i].append,
                           on_finish=lambda r, u, i=i: fins.__setitem__(i, (r, u))))
    sch.run_until_idle(10000)
    return outs, fins, sch


def test_single_vs_concurrent_greedy_identical(weights):
    prompts = _prompts(weights.cfg, 6)
    solo = [_run(weights, [p], max_batch=1)[0][0] for p in prompts]
    together, fins, sch = _run(weights, prompts, max_batch=4)
    assert together == solo
    assert all(f[0] == "length" and f[1]["completion_tokens"] == 12 for f in fins)
    assert sch.stats["admitted"] == 6 and not sch.lanes and sorted(sch.free_slots) == [0, 1, 2, 3]
    for s in range(4):          # invariant: cached token list length == tokens fed into the slot
        assert len(sch.slot_cache[s]) > 0


@pytest.mark.parametrize("depth", [2, 4, 8])
def test_mtp_chain_is_lossless(weights, depth):
    prompts = _prompts(weights.cfg, 2, seed=3)
    base = [_run(weights, [p], max_new=20, max_batch=1)[0][0] for p in prompts]
    for i, p in enumerate(prompts):
        outs, fins, sch = _run(weights, [p], max_new=20, max_batch=1, policy=MtpPolicy("on", depth=depth))
        assert outs[0] == base[i]
        assert sch.stats["mtp_steps"] > 0 and fins[0][1]["completion_tokens"] == 20


def test_mtp_tree_and_ngram_are_lossless(weights):
    p = [5, 6, 7, 8, 9, 5, 6, 7, 8, 9, 5, 6, 7, 8]      # repetitive prompt so the n-gram branch fires
    base = _run(weights, [p], max_new=16, max_batch=1)[0][0]
    outs, _, sch = _run(weights, [p], max_new=16, max_batch=1, policy=MtpPolicy("on", depth=4), ngram_draft=2,
                        tree_draft=True)
    assert outs[0] == base and sch.stats["tree_steps"] > 0
    outs, _, _ = _run(weights, [p], max_new=16, max_batch=1, policy=MtpPolicy("on", depth=4), ngram_draft=2)
    assert outs[0] == base


def test_forest_lanes_are_lossless(weights):
    prompts = _prompts(weights.cfg, 3, seed=5)
    base = [_run(weights, [p], max_new=10, max_batch=1)[0][0] for p in prompts]
    outs, _, sch = _run(weights, prompts, max_new=10, max_batch=4, policy=MtpPolicy("on", depth=4), mtp_lanes=True)
    assert outs == base and sch.stats["forest_steps"] > 0


def test_prefix_cache_live_and_checkpoint_hits(weights):
    cfg = weights.cfg
    p1 = _prompts(cfg, 1, seed=7, lo=20, hi=21)[0]
    orc = OracleModel(weights)
    sch = Scheduler(orc, 2, 128, eos_ids=[cfg.vocab_size - 1], policy=MtpPolicy("off"))
    out1 = []
    sch.submit(Request(p1, 6, GREEDY, ckpt_at=12, on_token=out1.append))
    sch.run_until_idle()
    # follow-up turn extends the whole first conversation: live hit on the same slot
    p2 = p1 + out1[:-1] + [3, 4, 5]
    out2 = []
    sch.submit(Request(p2, 5, GREEDY, on_token=out2.append))
    sch.run_until_idle()
    assert sch.stats["prefix_live"] == 1
    # a different continuation of the first 12 tokens on a fresh engine: checkpoint hit
    sch2 = Scheduler(OracleModel(weights), 2, 128, eos_ids=[cfg.vocab_size - 1], policy=MtpPolicy("off"))
    sch2.submit(Request(p1, 6, GREEDY, ckpt_at=12))
    sch2.run_until_idle()
    p3 = p1[:12] + [9, 9, 9, 9]
    out3 = []
    sch2.submit(Request(p3, 5, GREEDY, on_token=out3.append))
    sch2.run_until_idle()
    assert sch2.stats["prefix_ckpt"] == 1 and sch2.slot_ckpt_seq[0] == p1[:12]
    # every answer equals a cold run without any cache
    for p, o in ((p2, out2), (p3, out3)):
        cold, _, s2 = _run(weights, [p], max_new=5, max_batch=1, prefix_cache=False)
        assert cold[0] == o and s2.stats["prefix_miss"] == 1


def test_budget_eos_cancel_and_context_limit(weights):
    cfg = weights.cfg
    prompts = _prompts(cfg, 1, seed=9)
    base = _run(weights, prompts, max_new=8, max_batch=1)[0][0]
    stop = base[3]
    out, fins, _ = _run(weights, prompts, max_new=8, max_batch=1)
    assert len(out[0]) == 8
    orc = OracleModel(weights)
    sch = Scheduler(orc, 1, 128, eos_ids=[cfg.vocab_size - 1], policy=MtpPolicy("off"))
    got, fin = [], []
    sch.submit(Request(prompts[0], 8, GREEDY, stop_ids={stop}, on_token=got.append, on_finish=lambda r, u: fin.append(r)))
    sch.run_until_idle()
    assert got == base[:base.index(stop)] and fin == ["stop"]
    fin2 = []
    sch.submit(Request(list(range(200)), 8, GREEDY, on_finish=lambda r, u: fin2.append(r)))
    sch.run_until_idle()
    assert fin2 == ["context_length_exceeded"]
    req = Request(prompts[0], 50, GREEDY)
    sch.submit(req)
    sch.step(); sch.step()
    req.cancelled = True
    sch.run_until_idle()
    assert not sch.lanes and sch.free_slots == [0]


def test_seeded_sampling_is_reproducible_and_mtp_sample_runs(weights):
    prompts = _prompts(weights.cfg, 2, seed=11)
    sp = SamplingParams(temperature=0.9, top_p=0.9, top_k=20, seed=1234, repetition_penalty=1.1, presence_penalty=0.2)
    a = _run(weights, prompts, max_new=10, params=sp)[0]
    b = _run(weights, prompts, max_new=10, params=sp)[0]
    assert a == b
    c = _run(weights, prompts, max_new=10, params=SamplingParams(temperature=0.9, top_p=0.9, top_k=20, seed=99))[0]
    assert c != a
    d, fins, sch = _run(weights, prompts[:1], max_new=10, params=sp, max_batch=1, policy=MtpPolicy("on", depth=3))
    assert len(d[0]) == 10 and sch.stats["mtp_steps"] > 0


def test_moe_model_runs_through_scheduler():
    cfg = tiny_moe(mtp=False)
    w = ModelBuilder(cfg, SyntheticSource(cfg, 0, std=0.08), recipe="all").build()
    prompts = _prompts(cfg, 2, seed=13, lo=6, hi=12)
    solo = [_run(w, [p], max_new=6, max_batch=1)[0][0] for p in prompts]
    both = _run(w, prompts, max_new=6, max_batch=2)[0]
    assert both == solo


def test_policy_tuning_and_accept_rules():
    pol = MtpPolicy("auto", has_head=True)
    for _ in range(200):
        pol.record_step(3, 3, 4)            # everything accepted: deeper is better
    assert pol.active and pol.depth >= 4 and pol.yield_at(4) > 3.5
    bad = MtpPolicy("auto", has_head=True)
    for _ in range(200):
        bad.record_step(3, 0, 1)
    assert not bad.active
    for _ in range(5000):
        bad.tick()
    assert bad.active
    assert S.greedy_accept([5, 6, 7], [5, 6]) == 2 and S.greedy_accept([5, 9, 7], [5, 6]) == 1
    # tree: root(0) -> A chain 1,2 ; fork B: 3 (child of 0), 4 (child of 3)
    parent, toks = [-1, 0, 1, 0, 3], [10, 11, 12, 21, 22]
    assert S.tree_accept_walk(parent, toks, [11, 12, 0, 0, 0]) == [0, 1, 2]
    assert S.tree_accept_walk(parent, toks, [21, 0, 0, 22, 0]) == [0, 3, 4]
    assert S.tree_accept_walk(parent, toks, [99, 0, 0, 0, 0]) == [0]
    assert S.tree_accept_walk([-1, 0, 0], [1, 7, 7], [7, 0, 0]) == [0, 1]      # tie -> lowest child
    assert S.splitmix64(0) == 0xE220A8397B1DCDAF
    nuc = S.nucleus_host(torch.tensor([1.0, 3.0, 3.0, 0.5]), SamplingParams(temperature=1.0, top_k=3, top_p=0.99))
    assert nuc.ids[:2] == [1, 2] and abs(nuc.mass - sum(nuc.probs)) < 1e-6
    assert S.nucleus_host(torch.tensor([1.0, 3.0, 3.0]), SamplingParams(temperature=0.0)).ids == [1]
    toks_, cnts = S.penalty_list([1, 2, 2, 3, 2])
    assert toks_ == [2, 3, 1] and cnts == [3, 1, 1]


def test_log_lines_draft_log_and_accept_curve(weights, tmp_path, monkeypatch):
    """The [req] / [mtp] lines reach the given stream, every chain step lands in the JSONL draft log with the fed
    token, drafts, verify predictions and accepted count, and the accept-by-depth curve file follows the policy."""
    import io
    import json
    from velogb10_b200.engine import scheduler as sched_mod
    log_path, curve_path = tmp_path / "drafts.jsonl", tmp_path / "curve.json"
    monkeypatch.setenv("VELO_MTP_DRAFT_LOG", str(log_path))
    monkeypatch.setenv("VELO_MTP_CURVE_FILE", str(curve_path))
    monkeypatch.setattr(sched_mod, "MTP_LOG_EVERY", 5)
    stream = io.StringIO()
    prompts = _prompts(weights.cfg, 1, seed=3)
    base, _, _ = _run(weights, prompts, max_new=24, max_batch=1)
    outs, fins, sch = _run(weights, prompts, max_new=24, max_batch=1, policy=MtpPolicy("on", depth=3), log_stream=stream)
    assert outs == base
    text = stream.getvalue()
    assert "[req] 1 slot 0 prompt" in text and "prefix miss" in text and "temp 0.0" in text
    assert "done length generated 24" in text and "tok/s" in text
    assert "[mtp] steps 5 depth 3 acceptance" in text and "accept@k" in text
    assert list(sch.log)[-1].startswith("[req]")
    steps = [json.loads(l) for l in open(log_path)]
    assert len(steps) == sch.stats["mtp_steps"] > 0
    emitted = []
    for i, st in enumerate(steps):
        assert st["step"] == i + 1 and len(st["drafts"]) == 2 and len(st["preds"]) == 3 and 0 <= st["nacc"] <= 2
        assert st["drafts"][:st["nacc"]] == st["preds"][:st["nacc"]]           # accepted drafts match the verify
        emitted += st["preds"][:st["nacc"] + 1]
    assert outs[0][1:1 + len(emitted)] == emitted[:len(outs[0]) - 1]            # the log reproduces the emitted text
    curve = json.load(open(curve_path))
    assert curve["depth"] == 3 and curve["accept_by_depth"][0]["offered"] >= 5
    assert all(0.0 <= c["rate"] <= 1.0 and c["cond_chain"] <= c["rate"] + 1e-12 for c in curve["accept_by_depth"])
