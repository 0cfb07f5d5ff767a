"""Tiny hybrid model on the GPU runtime against the fp32 CPU oracle, plus the bitwise
batch-invariance / verify == sequential-decode gates."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _build(recipe="all", std=0.05, moe=False):
    from velogb10_b200.config import tiny_hybrid, tiny_moe
    from velogb10_b200.checkpoint.synthetic import SyntheticSource
    from velogb10_b200.models.weights import ModelBuilder
    cfg = tiny_moe() if moe else tiny_hybrid()
    w = ModelBuilder(cfg, SyntheticSource(cfg, 0, "cuda", std=std), recipe=recipe, device="cuda").build()
    return cfg, w


def _oracle(cfg, w):
    from velogb10_b200.models.oracle import OracleModel
    from velogb10_b200.checkpoint.synthetic import SyntheticSource
    from velogb10_b200.models.weights import ModelBuilder
    wc = ModelBuilder(cfg, SyntheticSource(cfg, 0, "cuda", std=0.05), recipe=w.recipe, device="cuda").build()
    return OracleModel(wc)


@pytest.mark.parametrize("recipe", ["all", "all,gdn:fp8", "off"])
def test_prefill_and_decode_match_oracle(recipe):
    from velogb10_b200.models.runtime import GpuModel
    cfg, w = _build(recipe)
    orc = _oracle(cfg, w)
    gm = GpuModel(w, keep_canonical=True)
    gm.alloc_state(4, 4 + 17, 256)
    orc.alloc_state(4, 4 + 17, 256)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (16,), generator=g).tolist()
    lg, _ = gm.prefill(1, prompt)
    lo, _ = orc.prefill(1, prompt)
    lg = lg.float().cpu()
    rel = (lg - lo).norm() / lo.norm()
    assert rel < 0.05, rel
    tok = int(lo.argmax())
    for i in range(4):
        lgd, _ = gm.decode([tok], [16 + i], [1])
        lod, _ = orc.decode([tok], [16 + i], [1])
        rel = (lgd[0].float().cpu() - lod[0]).norm() / lod[0].norm()
        assert rel < 0.05, (i, rel)
        tok = int(lod[0].argmax())


def test_batch_and_verify_are_bitwise_sequential():
    """Batch-4 decode == four single decodes; width-4 verify == 4 sequential decodes; checkpoints restore."""
    from velogb10_b200.models.runtime import GpuModel
    cfg, w = _build("all")
    gm = GpuModel(w, keep_canonical=True)
    gm.alloc_state(4, 4 + 17, 512)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (16, 23, 300, 260)]
    firsts = []
    for s, p in enumerate(prompts):
        lg, _ = gm.prefill(s, p)
        firsts.append(int(lg.argmax()))
    # snapshot state after prefill
    S0, C0, K0, V0 = gm.S.clone(), gm.conv.clone(), gm.kc.clone(), gm.vc.clone()
    pos = [len(p) for p in prompts]
    lb, _ = gm.decode(firsts, pos, [0, 1, 2, 3])
    lb = lb.clone()
    Sb = gm.S.clone()
    gm.S.copy_(S0); gm.conv.copy_(C0); gm.kc.copy_(K0); gm.vc.copy_(V0)
    for s in range(4):
        l1, _ = gm.decode([firsts[s]], [pos[s]], [s])
        assert torch.equal(l1[0], lb[s]), s
    assert torch.equal(gm.S, Sb)
    # chain verify on lane 2 (straddles the 256-key split boundary region) vs sequential decodes
    gm.S.copy_(S0); gm.conv.copy_(C0); gm.kc.copy_(K0); gm.vc.copy_(V0)
    toks = [firsts[2], 5, 7, 11]
    lv, _ = gm.verify(2, toks, pos[2], ckpt_base=4)
    lv = lv.clone()
    ck = [gm.S[:, 4 + t].clone() for t in range(4)]
    gm.S.copy_(S0); gm.conv.copy_(C0); gm.kc.copy_(K0); gm.vc.copy_(V0)
    for t in range(4):
        l1, _ = gm.decode([toks[t]], [pos[2] + t], [2])
        assert torch.equal(l1[0], lv[t]), t
        assert torch.equal(gm.S[:, 2], ck[t]), t


def test_graph_replay_matches_eager():
    from velogb10_b200.models.runtime import GpuModel
    cfg, w = _build("all")
    gm = GpuModel(w, keep_canonical=True)
    gm.alloc_state(2, 2 + 17, 128)
    gm.prefill(0, list(range(10, 30)))
    gm.prefill(1, list(range(40, 70)))
    S0, C0 = gm.S.clone(), gm.conv.clone()
    le, _ = gm.decode([3, 4], [20, 30], [0, 1])
    want = le.argmax(-1).int().clone()
    gm.S.copy_(S0); gm.conv.copy_(C0)
    got = gm.replay_decode([3, 4], [20, 30], [0, 1]).clone()
    gm.S.copy_(S0); gm.conv.copy_(C0)
    got2 = gm.replay_decode([3, 4], [20, 30], [0, 1]).clone()
    assert torch.equal(got, want) and torch.equal(got2, want)


def test_moe_model_matches_oracle_and_is_batch_invariant():
    """MoE FFN: per-pair decode path and sorted grouped prefill path against the oracle; verify == decode."""
    from velogb10_b200.models.runtime import GpuModel
    cfg, w = _build("all", moe=True)
    orc = _oracle(cfg, w)
    gm = GpuModel(w, keep_canonical=True)
    gm.alloc_state(2, 2 + 17, 256)
    orc.alloc_state(2, 2 + 17, 256)
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, cfg.vocab_size, (40,), generator=g).tolist()
    lg, _ = gm.prefill(0, prompt)          # 40 columns -> grouped path
    lo, _ = orc.prefill(0, prompt)
    rel = (lg.float().cpu() - lo).norm() / lo.norm()
    assert rel < 0.06, rel
    toks = [int(lo.argmax()), 3, 9, 27]
    S0, C0, K0, V0 = gm.S.clone(), gm.conv.clone(), gm.kc.clone(), gm.vc.clone()
    lv, _ = gm.verify(0, toks, 40, ckpt_base=2)
    lv = lv.clone()
    lov, _ = orc.verify(0, toks, 40, ckpt_base=2)
    assert ((lv.float().cpu() - lov).norm() / lov.norm()) < 0.06
    gm.S.copy_(S0); gm.conv.copy_(C0); gm.kc.copy_(K0); gm.vc.copy_(V0)
    for t in range(4):
        ld, _ = gm.decode([toks[t]], [40 + t], [0])
        assert torch.equal(ld[0], lv[t]), t


def test_draft_vocabulary_head_is_exact_subset(monkeypatch):
    """FR-Spec: the draft head scores a row subset of the real head; inside the subset the logits are those of
    the full head, outside it they are -inf."""
    from velogb10_b200.models.runtime import GpuModel
    from velogb10_b200.models.weights import draft_vocab_rows
    cfg, w_full = _build("all")
    _, w_sub = _build("all")
    monkeypatch.setenv("VELO_DRAFT_VOCAB", "0")
    full = GpuModel(w_full, keep_canonical=True)
    monkeypatch.setenv("VELO_DRAFT_VOCAB", "200")
    sub = GpuModel(w_sub, keep_canonical=True)
    assert full.draft_head is None and sub.draft_head is not None
    top, tail_start = draft_vocab_rows(200, cfg.vocab_size)
    assert (top + cfg.vocab_size - tail_start) % 128 == 0 and sub.draft_head.m == top + cfg.vocab_size - tail_start
    for m in (full, sub):
        m.alloc_state(2, 2 + 17, 256)
    prompt = list(range(3, 40))
    _, h1 = full.prefill(0, prompt)
    _, h2 = sub.prefill(0, prompt)
    assert torch.equal(h1, h2)
    toks, pos = [5, 9, 11], [37, 38, 39]
    lf, _ = full.mtp_forward(0, toks, h1[-3:], pos)
    lf = lf.clone()
    ls, _ = sub.mtp_forward(0, toks, h2[-3:], pos)
    ids = sub.draft_ids
    inside = torch.zeros(cfg.vocab_size, dtype=torch.bool, device="cuda")
    inside[ids] = True
    assert torch.isinf(ls[:, ~inside]).all() and (ls[:, ~inside] < 0).all()
    rel = ((ls[:, inside] - lf[:, inside]).norm() / lf[:, inside].norm()).item()
    assert rel < 2e-3, rel


def test_four_bit_kv_cache(monkeypatch):
    """--kv-cache q4: decode and tensor-core / scalar prefill over the 4-bit cache stay close to the bf16 cache,
    verify is still bit-identical to sequential decode, and the cache is 5 bits per value."""
    from velogb10_b200.models.runtime import GpuModel
    cfg, w1 = _build("all")
    _, w2 = _build("all")
    ref = GpuModel(w1, keep_canonical=True)
    monkeypatch.setenv("VELO_KV_QUANT", "q4")
    gm = GpuModel(w2, keep_canonical=True)
    assert gm.kv_q4 and not ref.kv_q4
    for m in (ref, gm):
        m.alloc_state(2, 2 + 17, 256)
    assert gm.kc.dtype == torch.uint8 and gm.kc.numel() * 8 + gm.ks.numel() * 16 == ref.kc.numel() * 5
    g = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, cfg.vocab_size, (150,), generator=g).tolist()
    l1, _ = ref.prefill(0, prompt)
    l2, _ = gm.prefill(0, prompt)
    rel = ((l2.float() - l1.float()).norm() / l1.float().norm()).item()
    assert rel < 0.08, rel
    toks = [int(l2.argmax()), 3, 9, 27]
    S0, C0 = gm.S.clone(), gm.conv.clone()
    kv0 = [t.clone() for t in gm._kv_tensors()]
    lv, _ = gm.verify(0, toks, 150, ckpt_base=2)
    lv = lv.clone()
    gm.S.copy_(S0); gm.conv.copy_(C0)
    for t, k in zip(gm._kv_tensors(), kv0):
        t.copy_(k)
    for t in range(4):
        ld, _ = gm.decode([toks[t]], [150 + t], [0])
        assert torch.equal(ld[0], lv[t]), t
    ld1, _ = ref.decode([toks[0]], [150], [0])
    gm.S.copy_(S0); gm.conv.copy_(C0)
    for t, k in zip(gm._kv_tensors(), kv0):
        t.copy_(k)
    ld2, _ = gm.decode([toks[0]], [150], [0])
    assert ((ld2.float() - ld1.float()).norm() / ld1.float().norm()).item() < 0.08


def test_debug_probes_print_and_do_not_change_results(monkeypatch, capfd):
    """VELO_DEBUG_HASH / VELO_CAP_DEBUG are host-side reads: the same prompt hashes the same twice, and logits are the
    ones of a run without the probes."""
    from velogb10_b200.checkpoint.synthetic import SyntheticSource
    from velogb10_b200.config import tiny_hybrid
    from velogb10_b200.models.runtime import GpuModel
    from velogb10_b200.models.weights import ModelBuilder
    cfg = tiny_hybrid(mtp=False)
    w = ModelBuilder(cfg, SyntheticSource(cfg, 0, "cuda", std=0.08), recipe="all", device="cuda").build()
    toks = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(2)).tolist()
    ref = GpuModel(w)
    ref.alloc_state(1, 20, 128)
    base = ref.prefill(0, toks)[0].clone()
    monkeypatch.setenv("VELO_DEBUG_HASH", "1")
    monkeypatch.setenv("VELO_CAP_DEBUG", "1")
    gm = GpuModel(w)
    gm.alloc_state(1, 20, 128)
    a = gm.prefill(0, toks)[0].clone()
    e1 = capfd.readouterr().err
    gm.zero_slot(0)
    b = gm.prefill(0, toks)[0].clone()
    e2 = capfd.readouterr().err
    assert torch.equal(a, base) and torch.equal(a, b)
    h1 = [l for l in e1.splitlines() if "[dbghash]" in l]
    assert len(h1) >= 3 and h1 == [l for l in e2.splitlines() if "[dbghash]" in l]
    assert "capdbg layer 0 normed" in e1 and "ffn out" in e1


def test_hy3_family_matches_oracle_and_verify_is_bitwise_sequential():
    """The attention-only ``hy_v3`` family on the CUDA runtime: sigmoid + bias router, ungated shared expert, plain
    norm weights, full-head rotary, bare q_proj, dense first layer, draft block: prefill / decode against the oracle,
    a chain verify equal to sequential decodes bit for bit, and lossless speculation through the scheduler."""
    from velogb10_b200.checkpoint.synthetic import SyntheticSource
    from velogb10_b200.config import tiny_hy3
    from velogb10_b200.engine.mtp import MtpPolicy
    from velogb10_b200.engine.sampling import SamplingParams
    from velogb10_b200.engine.scheduler import Request, Scheduler
    from velogb10_b200.models.oracle import OracleModel
    from velogb10_b200.models.runtime import GpuModel
    from velogb10_b200.models.weights import ModelBuilder
    from velogb10_b200.ops import lib
    cfg = tiny_hy3(mtp=True)
    recipe = "all,-router,-embed,-lmhead"
    w = ModelBuilder(cfg, SyntheticSource(cfg, 0, "cuda", std=0.08), recipe=recipe, device="cuda").build()
    orc = OracleModel(ModelBuilder(cfg, SyntheticSource(cfg, 0, "cuda", std=0.08), recipe=recipe, device="cuda").build())
    gm = GpuModel(w, keep_canonical=True)
    gm.alloc_state(2, 2 + 17, 256)
    orc.alloc_state(2, 2 + 17, 256)
    g = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, cfg.vocab_size, (40,), generator=g).tolist()
    lg, _ = gm.prefill(0, prompt)
    lo, _ = orc.prefill(0, prompt)
    assert ((lg.float().cpu() - lo).norm() / lo.norm()) < 0.06
    toks = [int(lo.argmax()), 3, 9, 27]
    K0, V0 = gm.kc.clone(), gm.vc.clone()
    lv, _ = gm.verify(0, toks, 40, ckpt_base=2)
    lv = lv.clone()
    lov, _ = orc.verify(0, toks, 40, ckpt_base=2)
    assert ((lv.float().cpu() - lov).norm() / lov.norm()) < 0.06
    gm.kc.copy_(K0); gm.vc.copy_(V0)
    for t in range(4):
        ld, _ = gm.decode([toks[t]], [40 + t], [0])
        assert torch.equal(ld[0], lv[t]), t

    def run(prompts, policy, max_batch):
        sch = Scheduler(gm, max_batch, 160, eos_ids=[cfg.vocab_size - 1], policy=policy)
        outs = [[] for _ in prompts]
        for i, p in enumerate(prompts):
            sch.submit(Request(p, 12, SamplingParams(temperature=0.0), on_token=outs[i].append))
        sch.run_until_idle(10000)
        torch.cuda.synchronize()
        lib.check_err_word()
        return outs, sch

    prompts = [torch.randint(0, cfg.vocab_size - 2, (int(n),), generator=g).tolist() for n in (9, 21, 14)]
    solo = [run([p], MtpPolicy("off", has_head=True), 1)[0][0] for p in prompts]
    together, sch = run(prompts, MtpPolicy("off", has_head=True), 4)
    assert together == solo and sch.stats.get("graph_steps", 0) > 0
    spec, sch = run(prompts[:2], MtpPolicy("on", depth=3), 1)
    assert spec == solo[:2] and sch.stats["mtp_steps"] > 0
