"""Checkpoint directories: reading (lazy safetensors source) and writing the quantized recipe layout.

Layout written by ``quantize_checkpoint`` (reference: src/main.rs:1605-1888): per quantized tensor
``stem`` = name minus ``.weight``

* NVFP4: ``stem.weight_packed`` U8 [M, K/2], ``stem.weight_scale`` F8_E4M3 [M, K/16],
  ``stem.weight_global_scale`` F32 [1] (reciprocal convention);
* FP8: ``stem.weight`` F8_E4M3 [M, K] + ``stem.weight_scale`` F32 [M];
* everything else copied through (norms, conv1d, A_log, dt_bias, vision tower, tensors whose last
  dim or row count is not a multiple of 16).

Stacked experts ``[E, M, K]`` are flattened to ``[E*M, K]``; per-expert un-fused checkpoints
(``…experts.<i>.{gate,up,down}_proj.weight``) are fused into ``…experts.gate_up_proj`` /
``…experts.down_proj`` first. Shards are capped (12 GB default), an index is written, sidecar files
are copied and ``config.json`` gets a ``quantization_config`` stamp.
"""
from __future__ import annotations

import json
import os
import re
import shutil
from typing import Dict, Iterable, List, Optional, Tuple

import torch
from safetensors import safe_open
from safetensors.torch import save_file

from ..models.weights import TensorSource
from ..quant import codec
from ..quant.recipe import fmt_for, parse_recipe

SIDECARS = ("tokenizer.json", "tokenizer_config.json", "generation_config.json", "chat_template.jinja",
            "merges.txt", "vocab.json", "preprocessor_config.json", "special_tokens_map.json")
INDEX = "model.safetensors.index.json"


def list_shards(model_dir: str) -> List[str]:
    idx = os.path.join(model_dir, INDEX)
    if os.path.exists(idx):
        with open(idx) as f:
            wm = json.load(f)["weight_map"]
        return [os.path.join(model_dir, s) for s in sorted(set(wm.values()))]
    return sorted(os.path.join(model_dir, n) for n in os.listdir(model_dir) if n.endswith(".safetensors"))


class SafetensorsSource(TensorSource):
    """Lazy tensor lookup over all shards of a checkpoint directory."""

    def __init__(self, model_dir: str, device: str = "cpu"):
        self.dir = model_dir
        self.device = device
        self.where: Dict[str, str] = {}
        self._open: Dict[str, object] = {}
        self.metadata: Dict[str, str] = {}
        for shard in list_shards(model_dir):
            with safe_open(shard, framework="pt", device="cpu") as f:
                for k in f.keys():
                    self.where[k] = shard
                self.metadata.update(f.metadata() or {})

    def names(self) -> List[str]:
        return list(self.where)

    def has(self, name: str) -> bool:
        return name in self.where

    def get(self, name: str) -> Optional[torch.Tensor]:
        shard = self.where.get(name)
        if shard is None:
            return None
        f = self._open.get(shard)
        if f is None:
            f = safe_open(shard, framework="pt", device="cpu")
            self._open[shard] = f
        return f.get_tensor(name)


# ------------------------------------------------------------------ writer

class ShardWriter:
    def __init__(self, out_dir: str, recipe: str, max_shard_bytes: int = 12 << 30):
        self.out, self.recipe, self.cap = out_dir, recipe, max_shard_bytes
        os.makedirs(out_dir, exist_ok=True)
        self.cur: Dict[str, torch.Tensor] = {}
        self.cur_bytes = 0
        self.files: List[Dict[str, torch.Tensor]] = []
        self.names: List[List[str]] = []
        self.total = 0

    def add(self, name: str, t: torch.Tensor):
        nb = t.numel() * t.element_size()
        if self.cur and self.cur_bytes + nb > self.cap:
            self._flush()
        self.cur[name] = t.contiguous().cpu()
        self.cur_bytes += nb
        self.total += nb

    def _flush(self):
        if not self.cur:
            return
        tmp = os.path.join(self.out, f".shard-{len(self.names):05d}.tmp")
        save_file(self.cur, tmp, metadata={"format": "pt", "quant_recipe": self.recipe})
        self.names.append(list(self.cur))
        self.cur, self.cur_bytes = {}, 0

    def finish(self):
        self._flush()
        n = len(self.names)
        if n == 1:
            os.replace(os.path.join(self.out, ".shard-00000.tmp"), os.path.join(self.out, "model.safetensors"))
            return
        wm = {}
        for i, names in enumerate(self.names):
            fn = f"model-{i + 1:05d}-of-{n:05d}.safetensors"
            os.replace(os.path.join(self.out, f".shard-{i:05d}.tmp"), os.path.join(self.out, fn))
            for k in names:
                wm[k] = fn
        with open(os.path.join(self.out, INDEX), "w") as f:
            json.dump({"metadata": {"total_size": self.total}, "weight_map": wm}, f, indent=1)


def emit_tensor(w: ShardWriter, name: str, t: torch.Tensor, recipe: Optional[dict], stats: dict):
    """Quantize-or-copy one tensor into the writer, honouring the recipe."""
    fmt = fmt_for(recipe, name)
    shape = tuple(t.shape)
    last = shape[-1] if shape else 0
    m_eff = shape[0] * shape[1] if len(shape) == 3 else (shape[0] if len(shape) == 2 else 0)
    ok = (fmt != "bf16" and len(shape) in (2, 3) and t.dtype == torch.bfloat16
          and last % codec.BLOCK == 0 and m_eff % 16 == 0 and ".visual." not in name)
    if not ok:
        w.add(name, t)
        stats["copied"] += 1
        return
    stem = name[:-len(".weight")] if name.endswith(".weight") else name
    w2 = t.reshape(m_eff, last)
    if fmt == "nvfp4":
        q = codec.quantize_nvfp4(w2)
        w.add(stem + ".weight_packed", q.packed)
        w.add(stem + ".weight_scale", q.scales.view(torch.float8_e4m3fn))
        w.add(stem + ".weight_global_scale", torch.tensor([q.global_scale], dtype=torch.float32))
        stats["nvfp4"] += 1
    else:
        q8 = codec.quantize_fp8(w2)
        w.add(stem + ".weight", q8.codes.view(torch.float8_e4m3fn))
        w.add(stem + ".weight_scale", q8.row_scale)
        stats["fp8"] += 1


_PER_EXPERT = re.compile(r"^(.*\.experts)\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")
_EXPERT_KINDS = ("gate_proj", "up_proj", "down_proj")


def _fuse_expert_set(base: str, d: Dict[Tuple[int, str], torch.Tensor], n: int):
    gu = torch.stack([torch.cat([d[(e, "gate_proj")], d[(e, "up_proj")]], 0) for e in range(n)], 0)
    dn = torch.stack([d[(e, "down_proj")] for e in range(n)], 0)
    return [(base + ".gate_up_proj", gu), (base + ".down_proj", dn)]


def _iter_fused(named: Iterable[Tuple[str, torch.Tensor]], n_experts: Optional[int] = None):
    """Pass tensors through, fusing per-expert 2-D tensors into stacked 3-D ones (gate‖up concatenated along
    rows; experts stacked in integer order). With ``n_experts`` known (from the checkpoint's config) a layer is
    fused, yielded and dropped as soon as its last tensor arrives, so the stash holds about one layer of experts
    (reference: src/main.rs ``run_quantize``); without it the count is only known once the input ends, and every
    per-expert tensor is held until then. An incomplete set is an error either way."""
    stash: Dict[str, Dict[Tuple[int, str], torch.Tensor]] = {}
    for name, t in named:
        mt = _PER_EXPERT.match(name)
        if not mt:
            yield name, t
            continue
        base, e, kind = mt.group(1), int(mt.group(2)), mt.group(3)
        d = stash.setdefault(base, {})
        d[(e, kind)] = t
        if n_experts and len(d) == 3 * n_experts and all((x, k) in d for x in range(n_experts) for k in _EXPERT_KINDS):
            yield from _fuse_expert_set(base, stash.pop(base), n_experts)
    for base, d in stash.items():
        n = n_experts or 1 + max(e for e, _ in d)
        missing = [(e, k) for e in range(n) for k in _EXPERT_KINDS if (e, k) not in d]
        if missing or len(d) != 3 * n:
            raise ValueError(f"{base}: incomplete or inconsistent per-expert set ({len(d)} tensors for {n} experts), "
                             f"missing {missing[:3]}")
        yield from _fuse_expert_set(base, d, n)


def write_checkpoint(out_dir: str, named: Iterable[Tuple[str, torch.Tensor]], config: dict,
                     recipe: str = "all,gdn:fp8", max_shard_bytes: int = 12 << 30,
                     sidecar_dir: Optional[str] = None) -> dict:
    """Write tensors in the recipe layout plus ``config.json``; returns counters."""
    rec = parse_recipe(recipe)
    w = ShardWriter(out_dir, recipe, max_shard_bytes)
    stats = {"nvfp4": 0, "fp8": 0, "copied": 0}
    tc = config.get("text_config", config)
    n_experts = tc.get("num_experts") or tc.get("n_routed_experts") or tc.get("num_local_experts")
    for name, t in _iter_fused(named, int(n_experts) if n_experts else None):
        emit_tensor(w, name, t, rec, stats)
    w.finish()
    cfg = dict(config)
    if rec is not None:
        cfg["quantization_config"] = {"quant_method": "compressed-tensors",
                                      "format": "nvfp4-pack-quantized", "recipe": recipe}
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    if sidecar_dir:
        for n in SIDECARS:
            p = os.path.join(sidecar_dir, n)
            if os.path.exists(p):
                shutil.copy(p, os.path.join(out_dir, n))
    stats["bytes"] = w.total
    return stats


def quantize_checkpoint(in_dir: str, out_dir: str, recipe: str = "all,gdn:fp8",
                        max_shard_bytes: int = 12 << 30) -> dict:
    """Offline quantizer: bf16 checkpoint directory -> recipe layout directory."""
    src = SafetensorsSource(in_dir)
    with open(os.path.join(in_dir, "config.json")) as f:
        config = json.load(f)
    named = ((n, src.get(n)) for n in src.names())
    return write_checkpoint(out_dir, named, config, recipe, max_shard_bytes, sidecar_dir=in_dir)


def requant_gdn(from_dir: str, out_dir: str, max_shard_bytes: int = 12 << 30) -> dict:
    """Derive a ``gdn4`` checkpoint from a mixed one: FP8 GDN in/out projections are decoded to bf16
    and re-encoded as NVFP4; every other tensor is copied verbatim (reference: src/main.rs:1897-1999)."""
    src = SafetensorsSource(from_dir)
    with open(os.path.join(from_dir, "config.json")) as f:
        config = json.load(f)
    w = ShardWriter(out_dir, "gdn4", max_shard_bytes)
    stats = {"requant": 0, "copied": 0}
    names = src.names()
    skip = set()
    for n in names:
        t = None
        if ".linear_attn." in n and n.endswith(".weight") and ("in_proj" in n or "out_proj" in n):
            t = src.get(n)
            if t.dtype == torch.float8_e4m3fn and t.dim() == 2 and t.shape[0] % 16 == 0 and t.shape[1] % 16 == 0:
                stem = n[:-len(".weight")]
                rs = src.get(stem + ".weight_scale").float()
                bf = codec.dequantize_fp8(t.view(torch.uint8), rs)
                q = codec.quantize_nvfp4(bf)
                w.add(stem + ".weight_packed", q.packed)
                w.add(stem + ".weight_scale", q.scales.view(torch.float8_e4m3fn))
                w.add(stem + ".weight_global_scale", torch.tensor([q.global_scale], dtype=torch.float32))
                skip.add(stem + ".weight_scale")
                skip.add(n)
                stats["requant"] += 1
    for n in names:
        if n in skip:
            continue
        w.add(n, src.get(n))
        stats["copied"] += 1
    w.finish()
    config.setdefault("quantization_config", {"quant_method": "compressed-tensors",
                                              "format": "nvfp4-pack-quantized"})["recipe"] = "gdn4"
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    for sn in SIDECARS:
        p = os.path.join(from_dir, sn)
        if os.path.exists(p):
            shutil.copy(p, os.path.join(out_dir, sn))
    return stats
