"""Seeded synthetic checkpoints: every tensor of a config drawn from N(0, 0.02).

Each tensor's values depend only on ``(seed, tensor name)``, never on generation order, so any
rank, any test and the CPU oracle see the same model. ``SyntheticSource`` produces tensors lazily on
the requested device, which lets a 27B-shaped model be built one tensor at a time without ever
holding the bf16 model in memory.
"""
from __future__ import annotations

import zlib
from typing import Dict, List, Optional, Tuple

import torch

from ..config import ModelConfig
from ..models.weights import PREFIX, TensorSource

STD = 0.02


def tensor_shapes(cfg: ModelConfig) -> Dict[str, Tuple[int, ...]]:
    """Unprefixed tensor name -> shape, in checkpoint naming (reference: src/gpu.rs:1221-1299)."""
    c = cfg
    h = c.hidden_size
    s: Dict[str, Tuple[int, ...]] = {"embed_tokens.weight": (c.vocab_size, h), "norm.weight": (h,)}
    if not c.tie_word_embeddings:
        s["lm_head.weight"] = (c.vocab_size, h)

    def layer(pre: str, i: int, full: bool):
        s[pre + "input_layernorm.weight"] = (h,)
        s[pre + "post_attention_layernorm.weight"] = (h,)
        if full:
            a = pre + "self_attn."
            s[a + "q_proj.weight"] = (c.q_out, h)
            s[a + "k_proj.weight"] = (c.kv_out, h)
            s[a + "v_proj.weight"] = (c.kv_out, h)
            s[a + "o_proj.weight"] = (h, c.num_heads * c.head_dim)
            s[a + "q_norm.weight"] = (c.head_dim,)
            s[a + "k_norm.weight"] = (c.head_dim,)
        else:
            g = pre + "linear_attn."
            s[g + "in_proj_qkv.weight"] = (c.conv_dim, h)
            s[g + "in_proj_z.weight"] = (c.value_dim, h)
            s[g + "in_proj_b.weight"] = (c.lin_num_v_heads, h)
            s[g + "in_proj_a.weight"] = (c.lin_num_v_heads, h)
            s[g + "conv1d.weight"] = (c.conv_dim, 1, c.conv_kernel)
            s[g + "A_log"] = (c.lin_num_v_heads,)
            s[g + "dt_bias"] = (c.lin_num_v_heads,)
            s[g + "norm.weight"] = (c.lin_v_dim,)
            s[g + "out_proj.weight"] = (h, c.value_dim)
        m = pre + "mlp."
        if c.is_moe_layer(i):
            E, I = c.num_experts, c.moe_intermediate_size
            hy3 = c.family == "hy_v3"
            # hy_v3 names the router and the (ungated) shared expert differently and adds a selection bias
            # (reference: src/gpu.rs:1151-1197)
            s[m + ("router.gate.weight" if hy3 else "gate.weight")] = (E, h)
            if hy3 and c.router_expert_bias:
                s[m + "expert_bias"] = (E,)
            s[m + "experts.gate_up_proj"] = (E, 2 * I, h)
            s[m + "experts.down_proj"] = (E, h, I)
            if c.shared_expert_intermediate_size > 0:
                si = c.shared_expert_intermediate_size
                sh = m + ("shared_mlp." if hy3 else "shared_expert.")
                s[sh + "gate_proj.weight"] = (si, h)
                s[sh + "up_proj.weight"] = (si, h)
                s[sh + "down_proj.weight"] = (h, si)
                if not hy3:
                    s[m + "shared_expert_gate.weight"] = (1, h)
        else:
            I = c.intermediate_size
            s[m + "gate_proj.weight"] = (I, h)
            s[m + "up_proj.weight"] = (I, h)
            s[m + "down_proj.weight"] = (h, I)

    for i in range(c.num_layers):
        layer(f"layers.{i}.", i, c.is_full_attn(i))
    if c.mtp_layers > 0 and c.family == "hy_v3":
        # the draft block is one more decoder layer after the last (reference: src/gpu.rs:1262-1283)
        mp = f"layers.{c.num_layers}."
        s[mp + "eh_proj.weight"] = (h, 2 * h)
        s[mp + "hnorm.weight"] = (h,)
        s[mp + "enorm.weight"] = (h,)
        s[mp + "final_layernorm.weight"] = (h,)
        layer(mp, -1, True)
    elif c.mtp_layers > 0:
        s["mtp.fc.weight"] = (h, 2 * h)
        s["mtp.pre_fc_norm_hidden.weight"] = (h,)
        s["mtp.pre_fc_norm_embedding.weight"] = (h,)
        s["mtp.norm.weight"] = (h,)
        layer("mtp.layers.0.", -1, True)
    return s


class SyntheticSource(TensorSource):
    def __init__(self, cfg: ModelConfig, seed: int = 0, device="cpu", std: float = STD):
        self.cfg, self.seed, self.device, self.std = cfg, seed, torch.device(device), std
        self.shapes = tensor_shapes(cfg)

    def _key(self, name: str) -> Optional[str]:
        for p in (PREFIX, "model."):
            if name.startswith(p):
                name = name[len(p):]
                break
        return name if name in self.shapes else None

    def has(self, name: str) -> bool:
        return self._key(name) is not None

    def names(self) -> List[str]:
        return list(self.shapes)

    def get(self, name: str) -> Optional[torch.Tensor]:
        key = self._key(name)
        if key is None:
            return None
        shape = self.shapes[key]
        g = torch.Generator(device=self.device)
        g.manual_seed((zlib.crc32(key.encode()) ^ (self.seed * 0x9E3779B1)) & 0x7FFFFFFF)
        n = 1
        for d in shape:
            n *= d
        # Generate in fp32 chunks and round to bf16 to bound the transient for vocabulary-sized tensors.
        out = torch.empty(n, dtype=torch.bfloat16, device=self.device)
        step = 1 << 26
        for o in range(0, n, step):
            e = min(n, o + step)
            out[o:e] = (torch.randn(e - o, generator=g, device=self.device, dtype=torch.float32) * self.std
                        ).to(torch.bfloat16)
        if self.cfg.family == "hy_v3" and "norm" in key and key.endswith(".weight"):
            out = (out.float() + 1.0).to(torch.bfloat16)     # plain (not zero-centred) RMSNorm weights in this family
        return out.reshape(shape)


def synthetic_state_dict(cfg: ModelConfig, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
    """The full bf16 model as a prefixed state dict (small configs only)."""
    src = SyntheticSource(cfg, seed, device)
    # MTP tensors are stored unprefixed (``mtp.fc.weight``), everything else under the language-model prefix
    pre = "model." if cfg.family == "hy_v3" else PREFIX
    return {(n if n.startswith("mtp.") else pre + n): src.get(n) for n in src.names()}
