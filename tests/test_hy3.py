"""The ``hy_v3`` model family (attention-only MoE: root-level config, sigmoid + selection-bias router, ungated shared
expert, plain RMSNorm weights, full-head rotary, bare q_proj, draft block stored as one more decoder layer) on the fp32
CPU oracle: config detection, router rule, checkpoint round trip in the family's recipe, and lossless scheduling."""
import json
import os

import torch

from velogb10_b200.checkpoint import io
from velogb10_b200.checkpoint.synthetic import SyntheticSource, synthetic_state_dict
from velogb10_b200.config import ModelConfig, tiny_hy3
from velogb10_b200.engine.mtp import MtpPolicy
from velogb10_b200.engine.sampling import SamplingParams
from velogb10_b200.engine.scheduler import Request, Scheduler
from velogb10_b200.models.oracle import OracleModel, router_topk
from velogb10_b200.models.weights import ModelBuilder

RECIPE = "all,-router,-embed,-lmhead"


def test_config_detection_from_a_root_level_config():
    raw = {"model_type": "hy_v3", "hidden_size": 256, "num_hidden_layers": 5, "num_attention_heads": 8,
           "num_key_value_heads": 2, "head_dim": 32, "vocab_size": 512, "intermediate_size": 640, "num_experts": 8,
           "num_experts_per_tok": 2, "moe_intermediate_size": 96, "num_shared_experts": 2, "first_k_dense_replace": 1,
           "qk_norm": True, "moe_router_use_sigmoid": True, "moe_router_enable_expert_bias": True, "route_norm": True,
           "router_scaling_factor": 2.826, "enable_lm_head_fp32": True, "tie_word_embeddings": False,
           "rope_parameters": {"rope_theta": 5e5}}
    c = ModelConfig.from_dict(raw)
    assert c.family == "hy_v3" and c.layer_types == ["full_attention"] * 5 and c.rotary_dim == c.head_dim == 32
    assert not c.attn_out_gate and c.q_out == 8 * 32 and c.qk_norm
    assert c.mlp_only_layers == [0] and not c.is_moe_layer(0) and c.is_moe_layer(1)
    assert c.shared_expert_intermediate_size == 192          # moe width x shared experts when the field is absent
    assert c.router_sigmoid and c.router_expert_bias and abs(c.router_scaling - 2.826) < 1e-6 and c.lm_head_fp32
    c2 = ModelConfig.from_dict(tiny_hy3().to_hf_dict())
    assert c2.asdict() == tiny_hy3().asdict()


def test_sigmoid_bias_router_rule():
    """Selection by sigmoid + bias, weights from the unbiased sigmoid, renormalised, scaled; ties go to the lower
    index (reference: tests/hy3_router_test.rs)."""
    cfg = tiny_hy3()
    logits = torch.tensor([0.0, 2.0, -1.0, 2.0, 0.5, 0.5, -3.0, 1.0] + [-9.0] * 8)
    bias = torch.zeros(16)
    bias[6] = 5.0                                           # a poor expert the bias pushes into the selection
    ids, w = router_topk(logits, 4, cfg, bias)
    assert ids.tolist() == [6, 1, 3, 7]
    s = torch.sigmoid(logits[ids])
    assert torch.allclose(w, s / s.sum() * 2.826, atol=1e-6) and abs(float(w.sum()) - 2.826) < 1e-5
    tie, _ = router_topk(torch.zeros(16), 4, cfg, torch.zeros(16))
    assert tie.tolist() == [0, 1, 2, 3]


def _run(w, prompts, policy, max_new=14, max_batch=4, **kw):
    sch = Scheduler(OracleModel(w), max_batch, 128, eos_ids=[w.cfg.vocab_size - 1], policy=policy, **kw)
    outs = [[] for _ in prompts]
    for i, p in enumerate(prompts):
        sch.submit(Request(p, max_new, SamplingParams(temperature=0.0), on_token=outs[i].append))
    sch.run_until_idle(10000)
    return outs, sch


def test_checkpoint_roundtrip_and_lossless_scheduling(tmp_path):
    cfg = tiny_hy3(mtp=True)
    sd = synthetic_state_dict(cfg, seed=0)
    assert "model.layers.1.mlp.router.gate.weight" in sd and "model.layers.1.mlp.expert_bias" in sd
    assert "model.layers.1.mlp.shared_mlp.down_proj.weight" in sd and "model.layers.3.eh_proj.weight" in sd
    assert not any("shared_expert_gate" in k or "linear_attn" in k for k in sd)
    out = str(tmp_path / "hy3")
    stats = io.write_checkpoint(out, sd.items(), cfg.to_hf_dict(), RECIPE)
    assert stats["nvfp4"] > 0
    conf = json.load(open(os.path.join(out, "config.json")))
    assert conf["model_type"] == "hy_v3" and "text_config" not in conf
    cfg2 = ModelConfig.from_json(os.path.join(out, "config.json"))
    src = io.SafetensorsSource(out)
    names = src.names()
    assert "model.layers.1.mlp.router.gate.weight" in names            # -router: left in bf16
    assert "model.embed_tokens.weight" in names and "model.layers.1.mlp.experts.gate_up_proj.weight_packed" in names
    w = ModelBuilder(cfg2, src).build()
    direct = ModelBuilder(cfg, SyntheticSource(cfg, 0), recipe=RECIPE).build()
    for (na, a), (nb, b) in zip(w.linears(), direct.linears()):
        assert na == nb and a.fmt == b.fmt and torch.equal(a.dequant(), b.dequant()), na
    assert w.mtp is not None and w.layers[0].mlp is not None and w.layers[1].moe.shared_gate is None
    assert abs(float(w.final_norm.mean())) < 0.05                      # plain weights near 1 held as w - 1
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size - 2, (int(n),), generator=g).tolist() for n in (9, 21, 14)]
    wide = ModelBuilder(cfg, SyntheticSource(cfg, 0, std=0.08), recipe=RECIPE).build()
    off = MtpPolicy("off", has_head=True)
    solo = [_run(wide, [p], off, max_batch=1)[0][0] for p in prompts]
    together, _ = _run(wide, prompts, off)
    assert together == solo
    spec, sch = _run(wide, prompts[:2], MtpPolicy("on", depth=3), max_batch=1)
    assert spec == solo[:2] and sch.stats["mtp_steps"] > 0
