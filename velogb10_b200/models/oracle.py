"""fp32 CPU oracle for the hybrid GatedDeltaNet + gated-GQA decoder (dense and MoE) and its MTP head.

This restates the model math in plain PyTorch, one token column at a time, and is the numerical
reference every CUDA kernel is compared against as well as the timed CPU baseline. The math follows
the reference's CPU forward (reference: src/qwen.rs:505-877) extended with what only its GPU path
has: key-head mapping for ``nk != nv`` (reference: kernels/gpu_batch.cu:540), the MoE block
(reference: src/gpu.rs:2199-2414), the MTP head (reference: src/gpu.rs:7875-7954), multi-column
verify with per-column state checkpoints and tree parents (reference: src/gpu.rs:4527-4947).

Every column is computed with matrix-vector products only, so a column's result is independent of
which other columns share the call: batch invariance holds by construction and the tests can use
exact equality to check the state plumbing (slots, positions, checkpoints) of the engine.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..config import ModelConfig
from .weights import AttnW, GdnW, LayerW, MlpW, ModelWeights, MoeW, QLinear


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, plus_one: bool = True) -> torch.Tensor:
    inv = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return x * inv * ((1.0 + w) if plus_one else w)


def rope_tables(cfg: ModelConfig, positions: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    half = cfg.rotary_dim // 2
    inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, half, dtype=torch.float32) * 2.0 / cfg.rotary_dim))
    ang = positions.float().unsqueeze(-1) * inv_freq
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rdim: int) -> torch.Tensor:
    """x [..., hd]; rotate-half on the first ``rdim`` dims; cos/sin [rdim/2]."""
    half = rdim // 2
    x1, x2 = x[..., :half], x[..., half:rdim]
    out = x.clone()
    out[..., :half] = x1 * cos - x2 * sin
    out[..., half:rdim] = x2 * cos + x1 * sin
    return out


def router_topk(logits: torch.Tensor, k: int, cfg: ModelConfig, bias: Optional[torch.Tensor] = None):
    """Expert selection + combine weights for one token (reference: kernels/gpu_batch.cu:3102-3240).

    softmax flavour: top-k of the logits (lowest index wins ties), weights ``exp(l-max)/sum_K``.
    sigmoid flavour: select by ``sigmoid(l)+bias``, weight by unbiased sigmoid, renormalise, scale.
    """
    E = logits.numel()
    if cfg.router_sigmoid:
        s = torch.sigmoid(logits)
        sel_score = s + (bias if (bias is not None and cfg.router_expert_bias) else 0.0)
    else:
        s = None
        sel_score = logits
    # stable descending order with lowest index first among ties
    order = sorted(range(E), key=lambda e: (-float(sel_score[e]), e))[:k]
    ids = torch.tensor(order, dtype=torch.long)
    if cfg.router_sigmoid:
        w = s[ids]
        if cfg.route_norm:
            w = w / w.sum()
        w = w * cfg.router_scaling
    else:
        l = logits[ids]
        e = torch.exp(l - l.max())
        w = e / e.sum()
    return ids, w


class _Deq:
    """Lazily dequantized fp32 copy of a QLinear."""

    def __init__(self):
        self.cache: Dict[int, torch.Tensor] = {}

    def __call__(self, q: QLinear) -> torch.Tensor:
        t = self.cache.get(id(q))
        if t is None:
            t = q.dequant(torch.float32).cpu()
            self.cache[id(q)] = t
        return t


@dataclass
class OracleState:
    k: Dict[int, torch.Tensor]          # layer -> [slots, nkv, max_seq, hd]
    v: Dict[int, torch.Tensor]
    S: Dict[int, torch.Tensor]          # layer -> [state_slots, nv, kd, vd]
    conv: Dict[int, torch.Tensor]       # layer -> [state_slots, conv_dim, ck]  (newest sample last)
    mtp_k: Optional[torch.Tensor] = None
    mtp_v: Optional[torch.Tensor] = None


class OracleModel:
    """Column-at-a-time fp32 forward. ``weights`` may hold quantized linears: they are dequantized
    once, so the oracle sees exactly the values the kernels decode."""

    def __init__(self, weights: ModelWeights, act_round: Optional[torch.dtype] = None):
        assert weights.tp_world == 1, "the oracle runs the unsharded model"
        self.w = weights
        self.cfg = weights.cfg
        self.deq = _Deq()
        self.state: Optional[OracleState] = None
        # Optional rounding of GEMM inputs/outputs to a 16-bit type, to mimic the device pipeline
        # when a tighter comparison is wanted. None = pure fp32.
        self.act_round = act_round

    # ---------------------------------------------------------------- state
    def alloc_state(self, n_slots: int, n_state_slots: int, max_seq: int):
        c = self.cfg
        k, v, S, conv = {}, {}, {}, {}
        for i in range(c.num_layers):
            if c.is_full_attn(i):
                k[i] = torch.zeros(n_slots, c.num_kv_heads, max_seq, c.head_dim)
                v[i] = torch.zeros(n_slots, c.num_kv_heads, max_seq, c.head_dim)
            else:
                S[i] = torch.zeros(n_state_slots, c.lin_num_v_heads, c.lin_k_dim, c.lin_v_dim)
                conv[i] = torch.zeros(n_state_slots, c.conv_dim, c.conv_kernel)
        st = OracleState(k, v, S, conv)
        if self.w.mtp is not None:
            st.mtp_k = torch.zeros(n_slots, c.num_kv_heads, max_seq, c.head_dim)
            st.mtp_v = torch.zeros(n_slots, c.num_kv_heads, max_seq, c.head_dim)
        self.state = st
        self.max_seq = max_seq
        return st

    def copy_state(self, src: int, dst: int):
        for i in self.state.S:
            self.state.S[i][dst] = self.state.S[i][src]
            self.state.conv[i][dst] = self.state.conv[i][src]

    def zero_slot(self, slot: int, zero_kv: bool = False):
        for i in self.state.S:
            self.state.S[i][slot].zero_()
            self.state.conv[i][slot].zero_()
        if zero_kv:
            for i in self.state.k:
                self.state.k[i][slot].zero_()
                self.state.v[i][slot].zero_()

    # ---------------------------------------------------------------- pieces
    def _rd(self, x):
        return x if self.act_round is None else x.to(self.act_round).float()

    def _mv(self, q: QLinear, x: torch.Tensor) -> torch.Tensor:
        return self._rd(torch.mv(self.deq(q), self._rd(x)))

    def embed(self, tok: int) -> torch.Tensor:
        # single-row dequant without materialising the table
        return self.w.embed.rows(tok, tok + 1).dequant(torch.bfloat16).float().cpu()[0]

    def attn(self, x, W: AttnW, kc, vc, slot: int, pos: int, key_pos: Optional[List[int]] = None):
        c = self.cfg
        nh, nkv, hd = c.num_heads, c.num_kv_heads, c.head_dim
        qkv = self._mv(W.qkv, x)
        qw = 2 * hd if c.attn_out_gate else hd
        qg = qkv[:nh * qw].reshape(nh, qw)
        q = qg[:, :hd]
        gate = qg[:, hd:] if c.attn_out_gate else None
        k = qkv[nh * qw:nh * qw + nkv * hd].reshape(nkv, hd)
        v = qkv[nh * qw + nkv * hd:].reshape(nkv, hd)
        cos, sin = rope_tables(c, torch.tensor(pos))
        q = apply_rope(rmsnorm(q, W.q_norm.cpu(), c.rms_eps), cos, sin, c.rotary_dim)
        k = apply_rope(rmsnorm(k, W.k_norm.cpu(), c.rms_eps), cos, sin, c.rotary_dim)
        kc[slot, :, pos] = self._rd(k)
        vc[slot, :, pos] = self._rd(v)
        q = self._rd(q)
        idx = torch.arange(pos + 1) if key_pos is None else torch.tensor(key_pos, dtype=torch.long)
        group = nh // nkv
        K = kc[slot][:, idx]                      # [nkv, T, hd]
        V = vc[slot][:, idx]
        qh = q.reshape(nkv, group, hd)
        s = torch.einsum("ngd,ntd->ngt", qh, K) / math.sqrt(hd)
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("ngt,ntd->ngd", p, V).reshape(nh, hd)
        if gate is not None:
            o = o * torch.sigmoid(gate)
        return self._mv(W.o, o.reshape(-1))

    def gdn(self, x, W: GdnW, S, conv, sslot: int):
        c = self.cfg
        nk, nv, kd, vd = c.lin_num_k_heads, c.lin_num_v_heads, c.lin_k_dim, c.lin_v_dim
        key_dim, value_dim, conv_dim = c.key_dim, c.value_dim, c.conv_dim
        proj = self._mv(W.in_proj, x)
        qkv = proj[:conv_dim]
        z = proj[conv_dim:conv_dim + value_dim].reshape(nv, vd)
        b = proj[conv_dim + value_dim:conv_dim + value_dim + nv]
        a = proj[conv_dim + value_dim + nv:conv_dim + value_dim + 2 * nv]
        st = conv[sslot]
        st[:, :-1] = st[:, 1:].clone()
        st[:, -1] = qkv
        acc = (W.conv_w.cpu() * st).sum(-1)
        qkv = F.silu(acc)
        q = qkv[:key_dim].reshape(nk, kd)
        k = qkv[key_dim:2 * key_dim].reshape(nk, kd)
        v = qkv[2 * key_dim:].reshape(nv, vd)
        q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) / math.sqrt(kd)
        k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
        beta = torch.sigmoid(b)
        g = torch.exp(-torch.exp(W.A_log.cpu()) * F.softplus(a + W.dt_bias.cpu()))
        hmap = torch.arange(nv) * nk // nv
        qv, kv = q[hmap], k[hmap]                                  # [nv, kd]
        Sl = S[sslot] * g.reshape(nv, 1, 1)
        kv_mem = torch.einsum("hkv,hk->hv", Sl, kv)
        delta = (v - kv_mem) * beta.unsqueeze(-1)
        Sl = Sl + torch.einsum("hk,hv->hkv", kv, delta)
        S[sslot] = Sl
        o = torch.einsum("hkv,hk->hv", Sl, qv)
        o = rmsnorm(o, W.norm.cpu(), c.rms_eps, plus_one=False) * F.silu(z)
        return self._mv(W.out, o.reshape(-1))

    def mlp(self, x, W: MlpW):
        gu = self._mv(W.gate_up, x)
        I = gu.numel() // 2
        return self._mv(W.down, self._rd(F.silu(gu[:I]) * gu[I:]))

    def moe(self, x, W: MoeW):
        c = self.cfg
        E, I, h = c.num_experts, c.moe_intermediate_size, c.hidden_size
        logits = torch.mv(self.deq(W.router), self._rd(x))
        ids, wts = router_topk(logits, c.num_experts_per_tok, c, None if W.expert_bias is None else W.expert_bias.cpu())
        gu_all, dn_all = self.deq(W.gate_up), self.deq(W.down)
        out = torch.zeros(h)
        xr = self._rd(x)
        for e, wt in zip(ids.tolist(), wts.tolist()):
            gu = self._rd(torch.mv(gu_all[e * 2 * I:(e + 1) * 2 * I], xr))
            hmid = self._rd(F.silu(gu[:I]) * gu[I:])
            out = out + wt * self._rd(torch.mv(dn_all[e * h:(e + 1) * h], hmid))
        if W.shared is not None:
            sh = self.mlp(x, W.shared)
            if W.shared_gate is not None:
                sh = sh * torch.sigmoid(torch.mv(self.deq(W.shared_gate), xr))
            out = out + sh
        return out

    def layer(self, x, L: LayerW, li, slot, sslot, pos, key_pos, kc=None, vc=None):
        c = self.cfg
        st = self.state
        n = self._rd(rmsnorm(x, L.input_norm.cpu(), c.rms_eps))
        if L.attn is not None:
            kc = st.k[li] if kc is None else kc
            vc = st.v[li] if vc is None else vc
            x = x + self.attn(n, L.attn, kc, vc, slot, pos, key_pos)
        else:
            x = x + self.gdn(n, L.gdn, st.S[li], st.conv[li], sslot)
        x = self._rd(x)
        n = self._rd(rmsnorm(x, L.post_norm.cpu(), c.rms_eps))
        x = x + (self.moe(n, L.moe) if L.moe is not None else self.mlp(n, L.mlp))
        return self._rd(x)

    def logits_from_hidden(self, hidden: torch.Tensor, norm_w: Optional[torch.Tensor] = None) -> torch.Tensor:
        nw = self.w.final_norm if norm_w is None else norm_w
        n = self._rd(rmsnorm(hidden, nw.cpu(), self.cfg.rms_eps))
        return torch.mv(self.deq(self.w.lm_head), n)

    # ---------------------------------------------------------------- column forward
    def forward_column(self, tok: int, pos: int, slot: int, sslot: Optional[int] = None,
                       key_pos: Optional[List[int]] = None, want_logits: bool = True):
        """One token through the backbone. Returns (logits [V] or None, pre-final-norm hidden [h])."""
        sslot = slot if sslot is None else sslot
        x = self._rd(self.embed(tok))
        for li, L in enumerate(self.w.layers):
            x = self.layer(x, L, li, slot, sslot, pos, key_pos)
        return (self.logits_from_hidden(x) if want_logits else None), x

    # ---------------------------------------------------------------- runner interface
    def prefill(self, slot: int, tokens: Sequence[int], pos_start: int = 0):
        """Sequential prefill of one lane. Returns (logits of the last token, hidden [N, h])."""
        hs = []
        logits = None
        for t, tok in enumerate(tokens):
            last = t == len(tokens) - 1
            logits, h = self.forward_column(int(tok), pos_start + t, slot, want_logits=last)
            hs.append(h)
        return logits, torch.stack(hs)

    def decode(self, tokens: Sequence[int], pos: Sequence[int], slots: Sequence[int]):
        """One token per lane. Returns (logits [B, V], hidden [B, h])."""
        outs = [self.forward_column(int(t), int(p), int(s)) for t, p, s in zip(tokens, pos, slots)]
        return torch.stack([o[0] for o in outs]), torch.stack([o[1] for o in outs])

    def verify(self, slot: int, tokens: Sequence[int], pos_start: int, ckpt_base: Optional[int] = None,
               parent: Optional[Sequence[int]] = None):
        """Width-N forward of one lane. Column t's recurrent state after the column is saved to
        state slot ``ckpt_base + t``. With ``parent`` (tree; parent[0] == -1, parents precede
        children) a column starts from its parent's checkpoint and attends only to the committed
        prefix plus its own ancestors; KV rows of column t live at position ``pos_start + t``.
        Returns (logits [N, V], hidden [N, h])."""
        n = len(tokens)
        logits, hs = [], []
        if parent is None:
            for t in range(n):
                l, h = self.forward_column(int(tokens[t]), pos_start + t, slot)
                if ckpt_base is not None:
                    self.copy_state(slot, ckpt_base + t)
                logits.append(l)
                hs.append(h)
            return torch.stack(logits), torch.stack(hs)
        assert ckpt_base is not None
        root_ckpt = ckpt_base + n          # scratch slot holding the pre-verify state
        self.copy_state(slot, root_ckpt)
        depth = [0] * n
        paths: List[List[int]] = []
        for t in range(n):
            p = parent[t]
            paths.append(([] if p < 0 else paths[p]) + [t])
            depth[t] = 0 if p < 0 else depth[p] + 1
        for t in range(n):
            p = parent[t]
            self.copy_state(root_ckpt if p < 0 else ckpt_base + p, slot)
            key_pos = list(range(pos_start)) + [pos_start + a for a in paths[t]]
            l, h = self._tree_column(int(tokens[t]), pos_start, t, depth[t], slot, key_pos)
            self.copy_state(slot, ckpt_base + t)
            logits.append(l)
            hs.append(h)
        return torch.stack(logits), torch.stack(hs)

    def _tree_column(self, tok, pos_start, col, depth, slot, key_pos):
        """A tree column has RoPE position ``pos_start + depth`` but stores KV at row ``pos_start + col``."""
        c = self.cfg
        x = self._rd(self.embed(tok))
        for li, L in enumerate(self.w.layers):
            if L.attn is not None:
                x = self._tree_attn_layer(x, L, li, slot, pos_start + depth, pos_start + col, key_pos)
            else:
                x = self.layer(x, L, li, slot, slot, 0, None)
        return self.logits_from_hidden(x), x

    def _tree_attn_layer(self, x, L, li, slot, rope_pos, row, key_pos):
        c = self.cfg
        st = self.state
        n = self._rd(rmsnorm(x, L.input_norm.cpu(), c.rms_eps))
        # write at `row` using rope position `rope_pos`: temporarily compute with pos=rope_pos into a
        # scratch row then move.
        kc, vc = st.k[li], st.v[li]
        save_k, save_v = kc[slot, :, rope_pos].clone(), vc[slot, :, rope_pos].clone()
        # compute K/V for this column
        W = L.attn
        nh, nkv, hd = c.num_heads, c.num_kv_heads, c.head_dim
        qkv = self._mv(W.qkv, n)
        qw = 2 * hd if c.attn_out_gate else hd
        qg = qkv[:nh * qw].reshape(nh, qw)
        q, gate = qg[:, :hd], (qg[:, hd:] if c.attn_out_gate else None)
        k = qkv[nh * qw:nh * qw + nkv * hd].reshape(nkv, hd)
        v = qkv[nh * qw + nkv * hd:].reshape(nkv, hd)
        cos, sin = rope_tables(c, torch.tensor(rope_pos))
        q = self._rd(apply_rope(rmsnorm(q, W.q_norm.cpu(), c.rms_eps), cos, sin, c.rotary_dim))
        k = apply_rope(rmsnorm(k, W.k_norm.cpu(), c.rms_eps), cos, sin, c.rotary_dim)
        kc[slot, :, rope_pos], vc[slot, :, rope_pos] = save_k, save_v
        kc[slot, :, row] = self._rd(k)
        vc[slot, :, row] = self._rd(v)
        idx = torch.tensor(key_pos, dtype=torch.long)
        group = nh // nkv
        K, V = kc[slot][:, idx], vc[slot][:, idx]
        s = torch.einsum("ngd,ntd->ngt", q.reshape(nkv, group, hd), K) / math.sqrt(hd)
        o = torch.einsum("ngt,ntd->ngd", torch.softmax(s, -1), V).reshape(nh, hd)
        if gate is not None:
            o = o * torch.sigmoid(gate)
        x = self._rd(x + self._mv(W.o, o.reshape(-1)))
        n2 = self._rd(rmsnorm(x, L.post_norm.cpu(), c.rms_eps))
        x = x + (self.moe(n2, L.moe) if L.moe is not None else self.mlp(n2, L.mlp))
        return self._rd(x)

    def verify_forest(self, lanes):
        """Several lanes' chain verifies in one call: list of (slot, tokens, pos_start, ckpt_base)."""
        return [self.verify(slot, toks, pos, ck) for slot, toks, pos, ck in lanes]

    def compact_kv(self, slot: int, pos_start: int, cols: Sequence[int]):
        """Move the KV rows of accepted tree columns to contiguous positions."""
        for li in self.state.k:
            for j, col in enumerate(cols):
                if col != j:
                    self.state.k[li][slot, :, pos_start + j] = self.state.k[li][slot, :, pos_start + col]
                    self.state.v[li][slot, :, pos_start + j] = self.state.v[li][slot, :, pos_start + col]

    # ---------------------------------------------------------------- MTP head
    def mtp_forward(self, slot: int, tokens: Sequence[int], hidden: torch.Tensor, pos: Sequence[int]):
        """Draft head over N (hidden_t, token_{t+1}) pairs of one lane, position ``pos[t]`` in the
        head's own KV cache. Returns (logits [N, V], head hidden [N, h])."""
        m = self.w.mtp
        c = self.cfg
        st = self.state
        outs, hs = [], []
        for t, tok in enumerate(tokens):
            e = self._rd(rmsnorm(self._rd(self.embed(int(tok))), m.norm_embed.cpu(), c.rms_eps))
            hh = self._rd(rmsnorm(self._rd(hidden[t].float()), m.norm_hidden.cpu(), c.rms_eps))
            x = self._mv(m.fc, torch.cat([e, hh]))
            x = self.layer(x, m.layer, -1, slot, slot, int(pos[t]), None, kc=st.mtp_k, vc=st.mtp_v)
            hs.append(x)
            outs.append(self.logits_from_hidden(x, m.norm))
        return torch.stack(outs), torch.stack(hs)
