"""Weight containers: canonical (checkpoint-order) quantized linears, fused per-layer groups, and
the builder that assembles a model from any tensor source (safetensors directory or the seeded
synthetic generator), with optional tensor-parallel sharding.

Canonical in-memory form of a linear ``[M, K]``:

* ``nvfp4``: ``packed`` u8 [M, K/2] (low nibble = even k), ``scales`` u8 [M, K/16] (E4M3 codes),
  ``row_scale`` f32 [M] holding ``1/global_scale`` of the segment each row came from, so tensors
  with different global scales can be fused along M (the reference keeps one scale per 16-row tile
  for the same purpose, reference: src/quant.rs:597-633).
* ``fp8``: ``codes`` u8 [M, K], ``row_scale`` f32 [M].
* ``bf16``: ``w`` bf16 [M, K].

The kernel-side tile-major layout is derived from this form by ``velogb10_b200.ops.gemm``.
"""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..config import ModelConfig
from ..quant import codec
from ..quant.recipe import fmt_for, parse_recipe


@dataclass
class QLinear:
    fmt: str
    m: int
    k: int
    packed: Optional[torch.Tensor] = None
    scales: Optional[torch.Tensor] = None
    codes: Optional[torch.Tensor] = None
    row_scale: Optional[torch.Tensor] = None
    w: Optional[torch.Tensor] = None
    kernel: object = None          # filled by ops.gemm.prepare()
    experts: int = 1               # >1: stacked experts, rows are [E * m_per_expert]

    # -- construction
    @classmethod
    def from_dense(cls, w: torch.Tensor, fmt: str) -> "QLinear":
        lead = w.shape[:-2]
        experts = int(lead[0]) if len(lead) == 1 else 1
        w2 = w.reshape(-1, w.shape[-1])
        m, k = w2.shape
        if fmt == "nvfp4" and (k % 16 != 0 or m % 16 != 0):
            fmt = "bf16"
        if fmt == "nvfp4":
            q = codec.quantize_nvfp4(w2)
            rs = torch.full((m,), 1.0, dtype=torch.float32, device=w.device) / q.global_scale
            return cls("nvfp4", m, k, packed=q.packed, scales=q.scales, row_scale=rs, experts=experts)
        if fmt == "fp8":
            q8 = codec.quantize_fp8(w2)
            return cls("fp8", m, k, codes=q8.codes, row_scale=q8.row_scale, experts=experts)
        return cls("bf16", m, k, w=w2.to(torch.bfloat16).contiguous(), experts=experts)

    # -- math
    def dequant(self, dtype=torch.float32) -> torch.Tensor:
        if self.fmt == "nvfp4":
            s = codec.e4m3_decode(self.scales) * self.row_scale.unsqueeze(-1)
            cd = torch.stack([self.packed & 0xF, self.packed >> 4], dim=-1).reshape(self.m, self.k)
            v = codec.e2m1_decode(cd).reshape(self.m, self.k // 16, 16) * s.unsqueeze(-1)
            return v.reshape(self.m, self.k).to(dtype)
        if self.fmt == "fp8":
            return (codec.e4m3_decode(self.codes) * self.row_scale.unsqueeze(-1)).to(dtype)
        return self.w.to(dtype)

    def to(self, device) -> "QLinear":
        def mv(t):
            return None if t is None else t.to(device)
        return QLinear(self.fmt, self.m, self.k, mv(self.packed), mv(self.scales), mv(self.codes),
                       mv(self.row_scale), mv(self.w), None, self.experts)

    # -- slicing (tensor parallel)
    def rows(self, r0: int, r1: int) -> "QLinear":
        def sl(t):
            return None if t is None else t[r0:r1].contiguous()
        return QLinear(self.fmt, r1 - r0, self.k, sl(self.packed), sl(self.scales), sl(self.codes),
                       sl(self.row_scale), sl(self.w), None, 1)

    def cols(self, k0: int, k1: int) -> "QLinear":
        assert k0 % 16 == 0 and k1 % 16 == 0
        q = QLinear(self.fmt, self.m, k1 - k0, row_scale=self.row_scale, experts=self.experts)
        if self.fmt == "nvfp4":
            q.packed = self.packed[:, k0 // 2:k1 // 2].contiguous()
            q.scales = self.scales[:, k0 // 16:k1 // 16].contiguous()
        elif self.fmt == "fp8":
            q.codes = self.codes[:, k0:k1].contiguous()
        else:
            q.w = self.w[:, k0:k1].contiguous()
        return q

    def nbytes(self) -> int:
        n = 0
        for t in (self.packed, self.scales, self.codes, self.row_scale, self.w):
            if t is not None:
                n += t.numel() * t.element_size()
        return n


def draft_vocab_rows(top: int, vocab: int, align: int = 128):
    """Row ranges of the smaller LM head the draft model scores (FR-Spec): the ``top`` lowest token ids (BPE
    ids are ordered by merge rank, i.e. by corpus frequency) plus the tail of the id range, where the special
    and added tokens live (a drafter that cannot propose the end-of-turn token cannot draft the end of a turn).
    ``top`` grows with real rows until the total is a multiple of ``align``; no padding rows (a zero row would
    score 0 and could win an arg-max against all-negative logits). Returns ``(top, tail_start)``
    (reference: src/quant.rs:697-721)."""
    tail = 512 if vocab >= 8192 else max(vocab // 8, 1)
    tail_start = max(vocab - tail, 0)
    top = min(max(top, 0), tail_start)
    while (top + (vocab - tail_start)) % align != 0 and top < tail_start:
        top += 1
    return top, tail_start


def fuse_rows(parts: List[QLinear]) -> QLinear:
    """Concatenate linears along M. All parts must share K and format; a format mismatch falls
    back to bf16 for the whole group."""
    k = parts[0].k
    assert all(p.k == k for p in parts)
    fmts = {p.fmt for p in parts}
    if len(fmts) > 1:
        return QLinear.from_dense(torch.cat([p.dequant(torch.bfloat16) for p in parts], 0), "bf16")
    fmt = parts[0].fmt
    cat = lambda name: torch.cat([getattr(p, name) for p in parts], 0)
    m = sum(p.m for p in parts)
    if fmt == "nvfp4":
        return QLinear(fmt, m, k, packed=cat("packed"), scales=cat("scales"), row_scale=cat("row_scale"))
    if fmt == "fp8":
        return QLinear(fmt, m, k, codes=cat("codes"), row_scale=cat("row_scale"))
    return QLinear(fmt, m, k, w=cat("w"))


# ------------------------------------------------------------------ per-layer groups

@dataclass
class AttnW:
    qkv: QLinear            # rows: [q|gate per head (nh*2hd), k (nkv*hd), v (nkv*hd)]
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    o: QLinear
    nh: int = 0             # local head counts (after TP sharding)
    nkv: int = 0


@dataclass
class GdnW:
    in_proj: QLinear        # rows: [q (key_dim), k (key_dim), v (value_dim), z (value_dim), b (nv), a (nv)]
    conv_w: torch.Tensor    # f32 [conv_dim, ck]
    A_log: torch.Tensor
    dt_bias: torch.Tensor
    norm: torch.Tensor      # f32 [vd]
    out: QLinear
    nk: int = 0
    nv: int = 0


@dataclass
class MlpW:
    gate_up: QLinear        # rows: [gate (I), up (I)]
    down: QLinear
    inter: int = 0


@dataclass
class MoeW:
    router: QLinear         # [E, h]
    gate_up: QLinear        # [E*2I, h], per expert [gate (I), up (I)]
    down: QLinear           # [E*h, I]
    shared: Optional[MlpW]
    shared_gate: Optional[QLinear]   # [1, h]
    expert_bias: Optional[torch.Tensor] = None
    n_local: int = 0        # experts resident on this rank
    e_base: int = 0         # first resident expert


@dataclass
class LayerW:
    input_norm: torch.Tensor
    post_norm: torch.Tensor
    attn: Optional[AttnW] = None
    gdn: Optional[GdnW] = None
    mlp: Optional[MlpW] = None
    moe: Optional[MoeW] = None


@dataclass
class MtpW:
    fc: QLinear                     # [h, 2h], input = [norm(embed) ; norm(hidden)]
    norm_hidden: torch.Tensor
    norm_embed: torch.Tensor
    layer: LayerW
    norm: torch.Tensor


@dataclass
class ModelWeights:
    cfg: ModelConfig
    embed: QLinear
    layers: List[LayerW]
    final_norm: torch.Tensor
    lm_head: QLinear
    mtp: Optional[MtpW] = None
    tp_rank: int = 0
    tp_world: int = 1
    recipe: str = "off"

    def linears(self):
        """Yield (name, QLinear) for every linear in the model."""
        yield "embed", self.embed
        if self.lm_head is not self.embed:
            yield "lm_head", self.lm_head
        layers = [(f"layers.{i}", l) for i, l in enumerate(self.layers)]
        if self.mtp is not None:
            yield "mtp.fc", self.mtp.fc
            layers.append(("mtp.layer", self.mtp.layer))
        for pre, l in layers:
            if l.attn:
                yield pre + ".attn.qkv", l.attn.qkv
                yield pre + ".attn.o", l.attn.o
            if l.gdn:
                yield pre + ".gdn.in_proj", l.gdn.in_proj
                yield pre + ".gdn.out", l.gdn.out
            if l.mlp:
                yield pre + ".mlp.gate_up", l.mlp.gate_up
                yield pre + ".mlp.down", l.mlp.down
            if l.moe:
                yield pre + ".moe.router", l.moe.router
                yield pre + ".moe.gate_up", l.moe.gate_up
                yield pre + ".moe.down", l.moe.down
                if l.moe.shared:
                    yield pre + ".moe.shared.gate_up", l.moe.shared.gate_up
                    yield pre + ".moe.shared.down", l.moe.shared.down
                if l.moe.shared_gate:
                    yield pre + ".moe.shared_gate", l.moe.shared_gate

    def weight_bytes(self) -> int:
        return sum(q.nbytes() for _, q in self.linears())


# ------------------------------------------------------------------ tensor sources

class TensorSource:
    """Name -> tensor lookup. ``get`` returns None when the tensor does not exist."""

    def get(self, name: str) -> Optional[torch.Tensor]:
        raise NotImplementedError

    def has(self, name: str) -> bool:
        return self.get(name) is not None


class DictSource(TensorSource):
    def __init__(self, tensors: Dict[str, torch.Tensor]):
        self.t = tensors

    def get(self, name):
        return self.t.get(name)

    def has(self, name):
        return name in self.t


PREFIX = "model.language_model."


class ModelBuilder:
    """Assembles ``ModelWeights`` from a tensor source.

    Accepts already-quantized groups (``.weight_packed/.weight_scale/.weight_global_scale`` or an
    F8 ``.weight`` + f32 ``.weight_scale``) and raw bf16 tensors, which are quantized on the fly
    when a recipe is given (the path synthetic models use). Mirrors the ingestion rules of the
    reference loader (reference: src/gpu.rs:787-976, :1221-1299) without its fragment repack.
    """

    def __init__(self, cfg: ModelConfig, src: TensorSource, recipe: str = "off", device="cpu",
                 tp_rank: int = 0, tp_world: int = 1, ep: bool = True):
        self.cfg, self.src, self.device = cfg, src, torch.device(device)
        self.recipe_str = recipe
        self.recipe = parse_recipe(recipe)
        self.rank, self.world = tp_rank, tp_world
        self.ep = ep
        # Debug loads (reference: src/gpu.rs:766-802, src/quant.rs:364-376):
        #  VELO_FAKE_QUANT=<recipe>   bf16 weights of the named groups are round-tripped through the 4- / 8-bit codec and
        #                             kept as bf16: the engine runs its bf16 path on values that carry the quantisation
        #                             error, which tells whether a group needs precision before committing a checkpoint;
        #  VELO_DEQUANT_AT_LOAD=1     quantised checkpoint tensors are decoded to bf16 at load: same numbers through the
        #                             bf16 kernels, to prove the quantised kernels against.
        self.fake_quant = parse_recipe(os.environ.get("VELO_FAKE_QUANT", "off"))
        self.dequant_at_load = os.environ.get("VELO_DEQUANT_AT_LOAD", "0") not in ("", "0")
        self.fake_quant_stats: List[Tuple[str, str, float]] = []       # (tensor, format, relative rms error)

    # -- raw access
    def _t(self, name: str) -> Optional[torch.Tensor]:
        for cand in (PREFIX + name, "model." + name, name):
            t = self.src.get(cand)
            if t is not None:
                return t
        return None

    def _f32(self, name: str) -> torch.Tensor:
        t = self._t(name)
        if t is None:
            raise KeyError(name)
        return t.to(self.device).float().contiguous()

    def _norm_w(self, name: str) -> torch.Tensor:
        """An RMSNorm weight in the zero-centred convention every norm kernel uses, ``y = x_hat * (1 + w)``. The
        ``hy_v3`` family stores plain weights (``y = x_hat * w``): they are held as ``w - 1`` (reference:
        src/gpu.rs:926-934), so kernels and oracle need no second flavour."""
        w = self._f32(name)
        return w - 1.0 if self.cfg.family == "hy_v3" else w

    def linear(self, stem: str, suffix: str = ".weight") -> QLinear:
        """Load one linear named ``stem`` (+``.weight`` for 2-D tensors; stacked experts have no
        suffix when unquantized)."""
        p = self._t(stem + ".weight_packed")
        if p is not None:
            sc = self._t(stem + ".weight_scale")
            gs = self._t(stem + ".weight_global_scale").float().reshape(-1)[0]
            experts = int(p.shape[0]) if p.dim() == 3 else 1
            p2 = p.reshape(-1, p.shape[-1]).to(self.device)
            sc2 = sc.reshape(-1, sc.shape[-1])
            if sc2.dtype != torch.uint8:
                sc2 = sc2.view(torch.uint8)
            m, k = p2.shape[0], p2.shape[1] * 2
            rs = torch.full((m,), 1.0, dtype=torch.float32, device=self.device) / float(gs)
            q = QLinear("nvfp4", m, k, packed=p2.contiguous(), scales=sc2.to(self.device).contiguous(),
                        row_scale=rs, experts=experts)
            return self._maybe_dequant(q)
        w = self._t(stem + suffix)
        if w is None and suffix:
            w = self._t(stem)
        if w is None:
            raise KeyError(stem)
        if w.dtype == torch.float8_e4m3fn:
            rs = self._t(stem + ".weight_scale").float().reshape(-1).to(self.device)
            experts = int(w.shape[0]) if w.dim() == 3 else 1
            c = w.view(torch.uint8).reshape(-1, w.shape[-1]).to(self.device)
            return self._maybe_dequant(QLinear("fp8", c.shape[0], c.shape[1], codes=c.contiguous(), row_scale=rs,
                                               experts=experts))
        fmt = fmt_for(self.recipe, stem + suffix)
        w = w.to(self.device)
        fq = fmt_for(self.fake_quant, stem + suffix) if self.fake_quant is not None else "bf16"
        if fq != "bf16" and w.dtype == torch.bfloat16:
            rt = QLinear.from_dense(w, fq)
            if rt.fmt == fq:
                back = rt.dequant(torch.float32).reshape(w.shape)
                err = float((back - w.float()).norm() / w.float().norm().clamp(min=1e-20))
                self.fake_quant_stats.append((stem + suffix, fq, err))
                return QLinear.from_dense(back.to(torch.bfloat16), "bf16")
        return QLinear.from_dense(w, fmt)

    def _maybe_dequant(self, q: QLinear) -> QLinear:
        if not self.dequant_at_load:
            return q
        w = q.dequant(torch.bfloat16)
        if q.experts > 1:
            w = w.reshape(q.experts, q.m // q.experts, q.k)
        return QLinear.from_dense(w, "bf16")

    # -- TP helpers
    def _shard_rows(self, q: QLinear, n_units: int, unit_rows: int) -> QLinear:
        """Keep this rank's contiguous share of ``n_units`` units of ``unit_rows`` rows."""
        if self.world == 1:
            return q
        per = n_units // self.world
        assert per * self.world == n_units, (n_units, self.world)
        r0 = self.rank * per * unit_rows
        return q.rows(r0, r0 + per * unit_rows)

    def _shard_cols(self, q: QLinear, n_units: int, unit_cols: int) -> QLinear:
        if self.world == 1:
            return q
        per = n_units // self.world
        assert per * self.world == n_units, (n_units, self.world)
        k0 = self.rank * per * unit_cols
        return q.cols(k0, k0 + per * unit_cols)

    # -- groups
    def attn(self, pre: str, shard: bool = True) -> AttnW:
        c = self.cfg
        q = self.linear(pre + "q_proj")
        k = self.linear(pre + "k_proj")
        v = self.linear(pre + "v_proj")
        o = self.linear(pre + "o_proj")
        nh, nkv, hd = c.num_heads, c.num_kv_heads, c.head_dim
        qw = 2 * hd if c.attn_out_gate else hd
        if shard and self.world > 1:
            w, r = self.world, self.rank
            assert nh % w == 0
            nh_l = nh // w
            q = q.rows(r * nh_l * qw, (r + 1) * nh_l * qw)
            o = o.cols(r * nh_l * hd, (r + 1) * nh_l * hd)
            if nkv >= w:
                assert nkv % w == 0
                nkv_l = nkv // w
                k0 = r * nkv_l
            else:   # more ranks than KV heads: each rank keeps the one head its q heads use
                nkv_l = 1
                k0 = (r * nh_l) // (nh // nkv)
                assert ((r + 1) * nh_l - 1) // (nh // nkv) == k0
            k = k.rows(k0 * hd, (k0 + nkv_l) * hd)
            v = v.rows(k0 * hd, (k0 + nkv_l) * hd)
            nh, nkv = nh_l, nkv_l
        if not c.qk_norm:
            raise NotImplementedError("attention without per-head q / k RMSNorm is not supported")
        return AttnW(fuse_rows([q, k, v]), self._norm_w(pre + "q_norm.weight"),
                     self._norm_w(pre + "k_norm.weight"), o, nh, nkv)

    def gdn(self, pre: str) -> GdnW:
        c = self.cfg
        nk, nv, kd, vd = c.lin_num_k_heads, c.lin_num_v_heads, c.lin_k_dim, c.lin_v_dim
        qkv = self.linear(pre + "in_proj_qkv")
        z = self.linear(pre + "in_proj_z")
        b = self.linear(pre + "in_proj_b")
        a = self.linear(pre + "in_proj_a")
        out = self.linear(pre + "out_proj")
        conv_w = self._f32(pre + "conv1d.weight").reshape(c.conv_dim, c.conv_kernel)
        A_log = self._f32(pre + "A_log")
        dt_bias = self._f32(pre + "dt_bias")
        key_dim, value_dim = c.key_dim, c.value_dim
        qs, ks, vs = qkv.rows(0, key_dim), qkv.rows(key_dim, 2 * key_dim), qkv.rows(2 * key_dim, c.conv_dim)
        cq, ck_, cv = conv_w[:key_dim], conv_w[key_dim:2 * key_dim], conv_w[2 * key_dim:]
        if self.world > 1:
            w, r = self.world, self.rank
            assert nk % w == 0 and nv % w == 0
            nk_l, nv_l = nk // w, nv // w
            qs = qs.rows(r * nk_l * kd, (r + 1) * nk_l * kd)
            ks = ks.rows(r * nk_l * kd, (r + 1) * nk_l * kd)
            vs = vs.rows(r * nv_l * vd, (r + 1) * nv_l * vd)
            z = z.rows(r * nv_l * vd, (r + 1) * nv_l * vd)
            b = b.rows(r * nv_l, (r + 1) * nv_l)
            a = a.rows(r * nv_l, (r + 1) * nv_l)
            out = out.cols(r * nv_l * vd, (r + 1) * nv_l * vd)
            cq = cq[r * nk_l * kd:(r + 1) * nk_l * kd]
            ck_ = ck_[r * nk_l * kd:(r + 1) * nk_l * kd]
            cv = cv[r * nv_l * vd:(r + 1) * nv_l * vd]
            A_log = A_log[r * nv_l:(r + 1) * nv_l].contiguous()
            dt_bias = dt_bias[r * nv_l:(r + 1) * nv_l].contiguous()
            nk, nv = nk_l, nv_l
        # b / a are tiny (nv rows) and rarely tile-aligned: carry them in bf16 inside the fused group
        # only when the group is bf16 anyway; otherwise requantize nothing and keep them as their own
        # rows of the fused tensor (the fused tensor falls back per-format in fuse_rows).
        parts = [qs, ks, vs, z, b, a]
        fm = {p.fmt for p in parts[:4]}
        if len(fm) == 1 and (b.fmt != qs.fmt or a.fmt != qs.fmt):
            tgt = qs.fmt
            b = QLinear.from_dense(_pad_rows(b.dequant(torch.bfloat16), 16), tgt)
            a = QLinear.from_dense(_pad_rows(a.dequant(torch.bfloat16), 16), tgt)
            b, a = b.rows(0, nv), a.rows(0, nv)
            parts = [qs, ks, vs, z, b, a]
        return GdnW(fuse_rows(parts), torch.cat([cq, ck_, cv], 0).contiguous(), A_log, dt_bias,
                    self._f32(pre + "norm.weight"), out, nk, nv)

    def mlp(self, pre: str, inter: int, shard: bool = True) -> MlpW:
        g = self.linear(pre + "gate_proj")
        u = self.linear(pre + "up_proj")
        d = self.linear(pre + "down_proj")
        if shard and self.world > 1:
            per = inter // self.world
            assert per * self.world == inter and per % 16 == 0
            r = self.rank
            g, u = g.rows(r * per, (r + 1) * per), u.rows(r * per, (r + 1) * per)
            d = d.cols(r * per, (r + 1) * per)
            inter = per
        return MlpW(fuse_rows([g, u]), d, inter)

    def moe(self, pre: str, shard: bool = True) -> MoeW:
        c = self.cfg
        E, I, h = c.num_experts, c.moe_intermediate_size, c.hidden_size
        hy3 = c.family == "hy_v3"
        router = self.linear(pre + ("router.gate" if hy3 else "gate"))
        if router.fmt != "bf16":
            router = QLinear.from_dense(router.dequant(torch.bfloat16), "bf16")
        gu = self.linear(pre + "experts.gate_up_proj", suffix="")
        dn = self.linear(pre + "experts.down_proj", suffix="")
        n_local, e_base = E, 0
        if shard and self.world > 1 and self.ep:
            assert E % self.world == 0
            n_local = E // self.world
            e_base = self.rank * n_local
            gu = gu.rows(e_base * 2 * I, (e_base + n_local) * 2 * I)
            dn = dn.rows(e_base * h, (e_base + n_local) * h)
        gu.experts = dn.experts = n_local
        shared = None
        sg = None
        sh = pre + ("shared_mlp." if hy3 else "shared_expert.")
        if c.shared_expert_intermediate_size > 0 and self._t(sh + "gate_proj.weight") is not None \
                or self._t(sh + "gate_proj.weight_packed") is not None:
            # under expert parallelism the shared expert is split like a dense tensor-parallel MLP: every rank adds its
            # partial (through the same gate) to its routed partial, and the one reduction of the layer sums both
            si = c.shared_expert_intermediate_size
            split = shard and self.world > 1 and self.ep and si % (16 * self.world) == 0
            shared = self.mlp(sh, si, shard=split)
            shared.partial = split
            if not hy3:                     # hy_v3 adds its shared expert ungated
                sgl = self.linear(pre + "shared_expert_gate")
                sg = sgl if sgl.fmt == "bf16" else QLinear.from_dense(sgl.dequant(torch.bfloat16), "bf16")
        bias = self._t(pre + "expert_bias")
        return MoeW(router, gu, dn, shared, sg, None if bias is None else bias.float().to(self.device),
                    n_local, e_base)

    def layer(self, pre: str, i: int, full: bool, shard: bool = True) -> LayerW:
        c = self.cfg
        lw = LayerW(self._norm_w(pre + "input_layernorm.weight"),
                    self._norm_w(pre + "post_attention_layernorm.weight"))
        if full:
            lw.attn = self.attn(pre + "self_attn.", shard)
        else:
            lw.gdn = self.gdn(pre + "linear_attn.")
        if c.is_moe_layer(i):
            lw.moe = self.moe(pre + "mlp.", shard)
        else:
            lw.mlp = self.mlp(pre + "mlp.", c.intermediate_size, shard)
        return lw

    def build(self) -> ModelWeights:
        c = self.cfg
        embed = self.linear("embed_tokens")
        layers = [self.layer(f"layers.{i}.", i, c.is_full_attn(i)) for i in range(c.num_layers)]
        final_norm = self._norm_w("norm.weight")
        if c.tie_word_embeddings or (self._t("lm_head.weight") is None
                                     and self._t("lm_head.weight_packed") is None):
            lm_head = embed
        else:
            lm_head = self.linear("lm_head")
        if self.world > 1:
            V = lm_head.m
            per = V // self.world
            assert per * self.world == V
            lm_head = lm_head.rows(self.rank * per, (self.rank + 1) * per)
        mtp = None
        hy3_mtp = f"layers.{c.num_layers}."
        if c.family == "hy_v3" and c.mtp_layers > 0 and (self._t(hy3_mtp + "eh_proj.weight") is not None
                                                          or self._t(hy3_mtp + "eh_proj.weight_packed") is not None):
            # hy_v3 keeps its draft block as decoder layer number num_layers: eh_proj = fc, hnorm / enorm = the two
            # input norms, final_layernorm = the head's norm (reference: src/gpu.rs:1262-1283); replicated on every rank
            mtp = MtpW(self.linear(hy3_mtp + "eh_proj"), self._norm_w(hy3_mtp + "hnorm.weight"),
                       self._norm_w(hy3_mtp + "enorm.weight"), self.layer(hy3_mtp, -1, True, shard=False),
                       self._norm_w(hy3_mtp + "final_layernorm.weight"))
        elif c.mtp_layers > 0 and (self._t("mtp.fc.weight") is not None
                                   or self._t("mtp.fc.weight_packed") is not None):
            # The draft head is replicated on every rank (reference: src/gpu.rs:2545-2547).
            mtp = MtpW(self.linear("mtp.fc"), self._f32("mtp.pre_fc_norm_hidden.weight"),
                       self._f32("mtp.pre_fc_norm_embedding.weight"),
                       self.layer("mtp.layers.0.", -1, True, shard=False), self._f32("mtp.norm.weight"))
        if self.fake_quant_stats and self.rank == 0:
            by_fmt: Dict[str, List[float]] = {}
            for _, f, e in self.fake_quant_stats:
                by_fmt.setdefault(f, []).append(e)
            print("[load] fake-quant: " + ", ".join(f"{len(v)} tensors through {f} (relative rms error mean "
                                                    f"{sum(v) / len(v):.4f}, max {max(v):.4f})" for f, v in by_fmt.items()),
                  file=sys.stderr)
        return ModelWeights(c, embed, layers, final_norm, lm_head, mtp, self.rank, self.world,
                            self.recipe_str)


def _pad_rows(w: torch.Tensor, mult: int) -> torch.Tensor:
    m = w.shape[0]
    pad = (-m) % mult
    if pad == 0:
        return w
    return torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)], 0)
