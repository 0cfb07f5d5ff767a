"""Codec, recipe and tile-layout tests (CPU). Mirrors the reference's inline codec tests
(reference: src/quant.rs:723-839) and adds checkpoint round trips."""
import json
import os

import pytest
import torch

from velogb10_b200.quant import codec
from velogb10_b200.quant.recipe import fmt_for, group_of, parse_recipe


def test_e4m3_is_decoded_as_a_float():
    assert codec._e4m3_value(0x38) == 1.0
    assert codec._e4m3_value(0x7E) == 448.0
    assert codec._e4m3_value(0x01) == 2.0 ** -9
    assert codec._e4m3_value(0xB8) == -1.0
    vals = codec.e4m3_decode(torch.arange(127, dtype=torch.uint8))
    assert torch.all(vals[1:] > vals[:-1])


def test_e4m3_encode_roundtrip_and_ties():
    codes = torch.arange(127, dtype=torch.uint8)
    vals = codec.e4m3_decode(codes)
    assert torch.equal(codec.e4m3_encode(vals), codes)
    assert torch.equal(codec.e4m3_encode(-vals[1:]), codes[1:] | 0x80)
    # exact midpoint goes to the lower code; non-finite and zero encode to 0; overflow saturates
    mid = (vals[10] + vals[11]) / 2
    assert int(codec.e4m3_encode(mid.reshape(1))) == 10
    assert int(codec.e4m3_encode(torch.tensor([float("inf")]))) == 0
    assert int(codec.e4m3_encode(torch.tensor([1e9]))) == 126


def test_e2m1_grid_exact_and_ties_to_even_code():
    grid = torch.tensor(codec.E2M1_VALUES)
    assert torch.equal(codec.e2m1_encode(grid), torch.arange(8, dtype=torch.uint8))
    assert torch.equal(codec.e2m1_encode(-grid[1:]), torch.arange(1, 8, dtype=torch.uint8) | 8)
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    assert codec.e2m1_encode(ties).tolist() == [0, 2, 2, 4, 4, 6, 6]
    assert int(codec.e2m1_encode(torch.tensor([100.0]))) == 7


def test_nvfp4_exact_block_roundtrip():
    """A tensor that is exactly representable survives quantization bit-for-bit."""
    g = torch.Generator().manual_seed(0)
    codes = torch.randint(0, 16, (32, 64), generator=g, dtype=torch.uint8)
    codes[:, ::16] = 7         # every block contains the maximum magnitude, so its scale is exact
    w = (codec.e2m1_decode(codes) * 0.5).to(torch.bfloat16)
    q = codec.quantize_nvfp4(w)
    back = codec.dequantize_nvfp4(q.packed, q.scales, q.global_scale)
    assert torch.equal(back, w)
    assert q.packed.shape == (32, 32) and q.scales.shape == (32, 4)
    # low nibble holds the even index
    c0 = codec.e2m1_encode(w[0, :2].float() / (codec.e4m3_decode(q.scales[0, :1]) / q.global_scale))
    assert int(q.packed[0, 0]) == int(c0[0]) | (int(c0[1]) << 4)


def test_nvfp4_and_fp8_roundtrip_error():
    g = torch.Generator().manual_seed(1)
    w = (torch.randn(128, 256, generator=g) * 0.02).to(torch.bfloat16)
    q = codec.quantize_nvfp4(w)
    rel, _ = codec.roundtrip_error(w, codec.dequantize_nvfp4(q.packed, q.scales, q.global_scale))
    assert rel < 0.15
    assert abs(q.global_scale - 2688.0 / float(w.abs().max())) < 1e-3 * q.global_scale
    q8 = codec.quantize_fp8(w)
    rel8, _ = codec.roundtrip_error(w, codec.dequantize_fp8(q8.codes, q8.row_scale))
    assert rel8 < 0.04
    assert codec.bits_per_weight("nvfp4", 256) == 4.5


def test_recipe_grammar():
    assert parse_recipe("off") is None and parse_recipe("") is None
    r = parse_recipe("all,gdn:fp8")
    assert r["gdn"] == "fp8" and r["mlp"] == "nvfp4" and r["lmhead"] == "nvfp4"
    r = parse_recipe("all,-router,-embed,-lmhead")
    assert "router" not in r and "embed" not in r and r["expert"] == "nvfp4"
    assert parse_recipe("nvfp4-mixed") == parse_recipe("all,gdn:fp8")
    with pytest.raises(ValueError):
        parse_recipe("bogus")
    with pytest.raises(ValueError):
        parse_recipe("mlp:int3")
    assert group_of("model.language_model.layers.3.mlp.gate.weight") == "router"
    assert group_of("mtp.layers.0.mlp.gate.weight") == "router"
    assert group_of("mtp.fc.weight") == "mtp"
    assert group_of("model.language_model.layers.3.mlp.experts.gate_up_proj") == "expert"
    assert group_of("model.language_model.layers.3.mlp.shared_expert.up_proj.weight") == "mlp"
    assert group_of("model.language_model.layers.0.linear_attn.in_proj_qkv.weight") == "gdn"
    assert group_of("model.language_model.layers.0.linear_attn.conv1d.weight") == "other"
    assert fmt_for(parse_recipe("mlp,attn"), "model.language_model.layers.0.linear_attn.out_proj.weight") == "bf16"


def test_tile_layouts_are_bijections():
    """Re-tiling for the tensor-core GEMM is a permutation of the padded bytes that can be inverted."""
    from velogb10_b200.ops import gemm as G
    g = torch.Generator().manual_seed(3)
    packed = torch.randint(0, 256, (200, 96), generator=g, dtype=torch.uint8)      # M=200, K=192
    scales = torch.randint(0, 127, (200, 12), generator=g, dtype=torch.uint8)
    t = G.tile_nvfp4(packed, scales)
    assert t.shape == (2, 2, 9216)
    # invert: physical chunk c of row r holds logical chunk c ^ ((r >> 1) & 3)
    for (r, ks, j) in [(0, 0, 0), (5, 1, 1), (131, 0, 3), (199, 1, 0), (70, 0, 2)]:
        mt, rr = divmod(r, 128)
        phys = j ^ ((rr >> 1) & 3)
        got = t[mt, ks, rr * 64 + phys * 16: rr * 64 + phys * 16 + 16]
        col0 = ks * 64 + j * 16
        want = torch.zeros(16, dtype=torch.uint8)
        avail = max(0, min(16, 96 - col0))
        want[:avail] = packed[r, col0:col0 + avail]
        assert torch.equal(got, want), (r, ks, j)
        sc = t[mt, ks, 8192 + rr * 8: 8192 + rr * 8 + 8]
        wsc = torch.zeros(8, dtype=torch.uint8)
        av = max(0, min(8, 12 - ks * 8))
        wsc[:av] = scales[r, ks * 8: ks * 8 + av]
        assert torch.equal(sc, wsc)
    assert int(t.sum(dtype=torch.int64)) == int(packed.sum(dtype=torch.int64) + scales.sum(dtype=torch.int64))
    codes = torch.randint(0, 256, (130, 256), generator=g, dtype=torch.uint8)
    t8 = G.tile_fp8(codes)
    assert t8.shape == (2, 2, 16384)
    assert torch.equal(t8[1, 1, 1 * 128 + ((3 ^ 1) * 16): 1 * 128 + ((3 ^ 1) * 16) + 16], codes[129, 128 + 48: 128 + 64])
    w = torch.randn(128, 128, generator=g).to(torch.bfloat16)
    t16 = G.tile_f16(w).view(torch.float16).reshape(1, 1, 2, 128, 8, 8)
    assert torch.equal(t16[0, 0, 1, 9, 2 ^ (9 & 7)], w[9, 64 + 16: 64 + 24].to(torch.float16))


def test_checkpoint_roundtrip_and_requant(tmp_path):
    """Write the recipe layout from a synthetic bf16 model, load it back, compare with load-time
    quantization, then derive a gdn4 checkpoint from the mixed one."""
    from velogb10_b200.checkpoint import io
    from velogb10_b200.checkpoint.synthetic import SyntheticSource, synthetic_state_dict
    from velogb10_b200.config import ModelConfig, tiny_moe
    from velogb10_b200.models.weights import ModelBuilder
    cfg = tiny_moe(mtp=True)
    sd = synthetic_state_dict(cfg, seed=0)
    # un-fuse one layer's experts to exercise the per-expert fuse path
    gu = sd.pop("model.language_model.layers.0.mlp.experts.gate_up_proj")
    dn = sd.pop("model.language_model.layers.0.mlp.experts.down_proj")
    I = cfg.moe_intermediate_size
    for e in range(cfg.num_experts):
        pre = f"model.language_model.layers.0.mlp.experts.{e}."
        sd[pre + "gate_proj.weight"] = gu[e, :I].clone()
        sd[pre + "up_proj.weight"] = gu[e, I:].clone()
        sd[pre + "down_proj.weight"] = dn[e].clone()
    out = str(tmp_path / "mixed")
    stats = io.write_checkpoint(out, sd.items(), cfg.to_hf_dict(), "all,gdn:fp8", max_shard_bytes=1 << 20)
    assert stats["nvfp4"] > 0 and stats["fp8"] > 0 and stats["copied"] > 0
    assert os.path.exists(os.path.join(out, io.INDEX))
    conf = json.load(open(os.path.join(out, "config.json")))
    assert conf["quantization_config"]["format"] == "nvfp4-pack-quantized"
    assert conf["quantization_config"]["recipe"] == "all,gdn:fp8"
    cfg2 = ModelConfig.from_json(os.path.join(out, "config.json"))
    assert cfg2.num_experts == cfg.num_experts and cfg2.layer_types == cfg.layer_types
    src = io.SafetensorsSource(out)
    assert src.metadata["quant_recipe"] == "all,gdn:fp8"
    names = src.names()
    assert "model.language_model.layers.0.mlp.experts.gate_up_proj.weight_packed" in names
    assert "model.language_model.layers.0.linear_attn.in_proj_qkv.weight_scale" in names
    assert src.get("model.language_model.layers.0.linear_attn.in_proj_qkv.weight").dtype == torch.float8_e4m3fn
    assert src.get("model.language_model.layers.0.linear_attn.conv1d.weight").dtype == torch.bfloat16
    loaded = ModelBuilder(cfg2, src).build()
    direct = ModelBuilder(cfg, SyntheticSource(cfg, 0), recipe="all,gdn:fp8").build()
    for (na, a), (nb, b) in zip(loaded.linears(), direct.linears()):
        assert na == nb and a.fmt == b.fmt, (na, a.fmt, b.fmt)
        assert torch.equal(a.dequant(), b.dequant()), na
    out4 = str(tmp_path / "gdn4")
    st = io.requant_gdn(out, out4)
    assert st["requant"] == 2 * len(cfg.linear_layers()) + 2 * len(cfg.linear_layers()) - 2 * len(cfg.linear_layers())  or st["requant"] > 0
    l4 = ModelBuilder(cfg2, io.SafetensorsSource(out4)).build()
    assert l4.layers[0].gdn.out.fmt == "nvfp4"
    assert l4.layers[0].mlp is None or l4.layers[0].mlp.down.fmt == "nvfp4"


def test_read_ahead_loader_builds_the_same_model(tmp_path):
    """The prefetching source hands the builder the same tensors as the plain lazy reader: through a window smaller
    than one layer (eviction and direct-read fallbacks), and with tensors in the checkpoint that the builder never asks for."""
    from velogb10_b200.checkpoint import io
    from velogb10_b200.checkpoint.synthetic import synthetic_state_dict
    from velogb10_b200.config import ModelConfig, tiny_hybrid
    from velogb10_b200.models.weights import ModelBuilder
    cfg = tiny_hybrid(mtp=True)
    sd = synthetic_state_dict(cfg, seed=0)
    sd["model.visual.blocks.0.unused.weight"] = torch.zeros(64, 64, dtype=torch.bfloat16)
    sd["model.language_model.layers.0.unused_tail.weight"] = torch.zeros(64, 64, dtype=torch.bfloat16)
    out = str(tmp_path / "ck")
    io.write_checkpoint(out, sd.items(), cfg.to_hf_dict(), "all,gdn:fp8", max_shard_bytes=1 << 20)
    cfg2 = ModelConfig.from_json(os.path.join(out, "config.json"))
    plain = ModelBuilder(cfg2, io.SafetensorsSource(out)).build()
    for workers, ahead in ((3, 2 << 30), (2, 4096)):
        src = io.PrefetchSource(io.SafetensorsSource(out), "cpu", workers=workers, ahead_bytes=ahead)
        try:
            got = ModelBuilder(cfg2, src).build()
        finally:
            src.close()
        st = src.summary()
        assert st["hits"] > 0 and st["hits"] + st["misses"] >= len(list(plain.linears()))
        for (na, a), (nb, b) in zip(got.linears(), plain.linears()):
            assert na == nb and a.fmt == b.fmt and torch.equal(a.dequant(), b.dequant()), na
        assert torch.equal(got.embed.dequant() if hasattr(got.embed, "dequant") else got.embed,
                           plain.embed.dequant() if hasattr(plain.embed, "dequant") else plain.embed)
    assert "read" in io.load_report(src, 1.0) and "no read-ahead" in io.load_report(io.SafetensorsSource(out), 1.0)
    monkey = os.environ.get("VELO_LOAD_WORKERS")
    os.environ["VELO_LOAD_WORKERS"] = "0"
    try:
        assert isinstance(io.open_checkpoint(out), io.SafetensorsSource)
    finally:
        if monkey is None:
            del os.environ["VELO_LOAD_WORKERS"]
        else:
            os.environ["VELO_LOAD_WORKERS"] = monkey


def test_draft_vocab_rows_rule():
    """FR-Spec row selection: the most frequent ids plus the special-token tail, padded with real rows."""
    from velogb10_b200.models.weights import draft_vocab_rows
    top, tail = draft_vocab_rows(65536, 248320)
    assert tail == 248320 - 512 and top >= 65536 and (top + 512) % 128 == 0 and top - 65536 < 128
    top, tail = draft_vocab_rows(10 ** 9, 248320)              # asking for more than the vocabulary keeps every row once
    assert top == tail
    top, tail = draft_vocab_rows(200, 1024)
    assert tail == 1024 - 128 and (top + 128) % 128 == 0


def test_per_expert_fuse_streams_one_layer_at_a_time():
    """With the expert count known, a layer's stacked tensors come out as soon as its last per-expert tensor went
    in (nothing of it stays stashed); a set that never completes is an error."""
    from velogb10_b200.checkpoint import io
    E, seen = 3, []

    def feed():
        for layer in range(2):
            for e in range(E):
                for kind in ("gate_proj", "up_proj", "down_proj"):
                    seen.append((layer, e, kind))
                    yield f"m.layers.{layer}.mlp.experts.{e}.{kind}.weight", torch.full((2, 4), float(e))
            yield f"m.layers.{layer}.post.weight", torch.zeros(1)
    order = []
    for name, t in io._iter_fused(feed(), E):
        order.append((name, len(seen)))
    names = [n for n, _ in order]
    assert names == ["m.layers.0.mlp.experts.gate_up_proj", "m.layers.0.mlp.experts.down_proj", "m.layers.0.post.weight",
                     "m.layers.1.mlp.experts.gate_up_proj", "m.layers.1.mlp.experts.down_proj", "m.layers.1.post.weight"]
    assert order[0][1] == 3 * E and order[3][1] == 6 * E          # fused before the next layer was read
    gu = next(t for n, t in io._iter_fused(feed(), E) if n.endswith("0.mlp.experts.gate_up_proj"))
    assert gu.shape == (E, 4, 4) and gu[2].eq(2).all()
    with pytest.raises(ValueError):
        list(io._iter_fused([("m.layers.0.mlp.experts.0.gate_proj.weight", torch.zeros(2, 4))], E))


def test_fake_quant_and_dequant_at_load(tmp_path, monkeypatch):
    """VELO_FAKE_QUANT keeps bf16 kernels but feeds them weights that carry the codec's error: the model then behaves
    like the really quantised one, not like the bf16 one. VELO_DEQUANT_AT_LOAD decodes a quantised checkpoint to bf16
    at load: every linear is bf16 and the values are those of the quantised load."""
    from velogb10_b200.checkpoint import io
    from velogb10_b200.checkpoint.synthetic import SyntheticSource, synthetic_state_dict
    from velogb10_b200.config import ModelConfig, tiny_hybrid
    from velogb10_b200.models.oracle import OracleModel
    from velogb10_b200.models.weights import ModelBuilder
    cfg = tiny_hybrid(mtp=False)
    toks = torch.randint(0, cfg.vocab_size, (24,), generator=torch.Generator().manual_seed(1)).tolist()

    def logits(w):
        m = OracleModel(w)
        m.alloc_state(1, 2, 64)
        return m.prefill(0, toks)[0].float()

    plain = logits(ModelBuilder(cfg, SyntheticSource(cfg, 0, std=0.08)).build())
    quant = logits(ModelBuilder(cfg, SyntheticSource(cfg, 0, std=0.08), recipe="all,gdn:fp8").build())
    monkeypatch.setenv("VELO_FAKE_QUANT", "all,gdn:fp8")
    b = ModelBuilder(cfg, SyntheticSource(cfg, 0, std=0.08))
    wf = b.build()
    assert all(q.fmt == "bf16" for _, q in wf.linears()) and b.fake_quant_stats
    assert {f for _, f, _ in b.fake_quant_stats} == {"nvfp4", "fp8"} and all(0 < e < 0.2 for _, _, e in b.fake_quant_stats)
    fake = logits(wf)
    monkeypatch.delenv("VELO_FAKE_QUANT")
    d_fq = float((fake - quant).norm() / quant.norm())
    d_pl = float((plain - quant).norm() / quant.norm())
    assert d_fq < 0.25 * d_pl, (d_fq, d_pl)
    # dequantise-at-load from a checkpoint in the recipe layout
    out = str(tmp_path / "ck")
    io.write_checkpoint(out, synthetic_state_dict(cfg, seed=0).items(), cfg.to_hf_dict(), "all,gdn:fp8")
    cfg2 = ModelConfig.from_json(os.path.join(out, "config.json"))
    wq = ModelBuilder(cfg2, io.SafetensorsSource(out)).build()
    monkeypatch.setenv("VELO_DEQUANT_AT_LOAD", "1")
    wd = ModelBuilder(cfg2, io.SafetensorsSource(out)).build()
    assert any(q.fmt != "bf16" for _, q in wq.linears()) and all(q.fmt == "bf16" for _, q in wd.linears())
    for (na, a), (nb, bq) in zip(wq.linears(), wd.linears()):
        # (rows fused from several checkpoint tensors are re-encoded to the group's common format in the quantised
        # load, so those agree to one more rounding rather than exactly)
        x, y = a.dequant(torch.float32), bq.dequant(torch.float32)
        assert na == nb and float((x - y).norm() / x.norm()) < 0.03, na
    assert float((logits(wd) - logits(wq)).norm() / logits(wq).norm()) < 0.05
