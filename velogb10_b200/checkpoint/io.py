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


class PrefetchSource(TensorSource):
    """Read-ahead in front of a ``SafetensorsSource``: worker threads walk the checkpoint in the order a model builder
    asks for it (embedding, layers by index, the rest), read each tensor into a pinned host buffer of their own and
    start its host->device copy on a side stream, at most ``ahead_bytes`` ahead of the consumer. ``get`` hands out the
    staged device tensor (the consumer's stream waits on the copy's event, the host does not) or reads directly for a
    name outside the predicted order. Disk reads, the pinned memcpy and the uploads therefore overlap the builder's
    GPU-side quantise / tile work; the counters split a load into read, wait and build time for the ``[load]`` line.
    Plays the part of the reference's record / replay assembly pipeline with its worker pool and single uploader
    (reference: src/gpu.rs:1304-1584), with the repack itself left to the GPU.

    On a CPU device the workers only read ahead (no pinned staging)."""

    _LAYER = re.compile(r"\.layers\.(\d+)\.")

    def __init__(self, inner: "SafetensorsSource", device="cpu", workers: int = 4, ahead_bytes: int = 2 << 30,
                 buf_bytes: int = 256 << 20):
        import threading
        self.inner, self.device = inner, torch.device(device)
        self.metadata = inner.metadata
        self.cuda = self.device.type == "cuda"
        self.stats = {"bytes": 0, "read_s": 0.0, "wait_s": 0.0, "hits": 0, "misses": 0, "direct_bytes": 0}
        self._order = sorted(inner.names(), key=self._rank)
        self._idx = {n: i for i, n in enumerate(self._order)}
        self._pending = set(self._order)
        self._staged: Dict[str, Tuple[torch.Tensor, object]] = {}
        self._cv = threading.Condition()
        self._next, self._inflight, self._ahead, self._buf_bytes = 0, 0, ahead_bytes, buf_bytes
        self._stop, self._failed = False, None
        for shard in set(inner.where.values()):             # ask the page cache to start on every shard now
            try:
                fd = os.open(shard, os.O_RDONLY)
                os.posix_fadvise(fd, 0, 0, os.POSIX_FADV_WILLNEED)
                os.close(fd)
            except (OSError, AttributeError):
                pass
        self._threads = [threading.Thread(target=self._work, daemon=True) for _ in range(max(1, workers))]
        for t in self._threads:
            t.start()

    def _rank(self, name: str):
        m = self._LAYER.search(name)
        if m:
            return (1 if ".mtp." not in name and not name.startswith("mtp.") else 3, int(m.group(1)), name)
        return (0 if "embed" in name else 2, 0, name)

    def _work(self):
        import time
        handles: Dict[str, object] = {}
        pinned = torch.empty(self._buf_bytes, dtype=torch.uint8).pin_memory() if self.cuda else None
        stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        busy = None                                          # event of the copy still reading this worker's buffer
        try:
            while True:
                with self._cv:
                    while not self._stop and self._next < len(self._order) and self._inflight >= self._ahead:
                        self._cv.wait(0.5)
                    if self._stop or self._next >= len(self._order):
                        return
                    name = self._order[self._next]
                    self._next += 1
                    if name not in self._pending:            # the consumer already read it directly
                        continue
                t0 = time.time()
                shard = self.inner.where[name]
                f = handles.get(shard)
                if f is None:
                    f = handles[shard] = safe_open(shard, framework="pt", device="cpu")
                t = f.get_tensor(name)
                nb = t.numel() * t.element_size()
                ev = None
                if self.cuda and 0 < nb <= self._buf_bytes:
                    if busy is not None:
                        busy.synchronize()
                    host = pinned[:nb].view(t.dtype).view(t.shape) if t.dtype != torch.bool else None
                    if host is not None:
                        host.copy_(t)
                        with torch.cuda.stream(stream):
                            t = torch.empty(t.shape, dtype=t.dtype, device=self.device)
                            t.copy_(host, non_blocking=True)
                            ev = busy = torch.cuda.Event()
                            ev.record(stream)
                with self._cv:
                    self.stats["read_s"] += time.time() - t0
                    self.stats["bytes"] += nb
                    if name in self._pending:
                        self._staged[name] = (t, ev)
                        self._inflight += nb
                    self._cv.notify_all()
        except Exception as e:  # noqa: BLE001 - reported to the consumer, which falls back to direct reads
            with self._cv:
                self._failed = e
                self._cv.notify_all()

    def names(self) -> List[str]:
        return self.inner.names()

    def has(self, name: str) -> bool:
        return self.inner.has(name)

    def get(self, name: str) -> Optional[torch.Tensor]:
        import time
        if not self.inner.has(name):
            return None
        t0 = time.time()
        with self._cv:
            if name in self._pending:
                # wait only for a tensor a worker has already claimed or is about to (its rank is near the cursor)
                while name not in self._staged and self._failed is None and not self._stop \
                        and self._claimed_or_near(name):
                    if self._inflight >= self._ahead and not self._drop_passed(name):
                        break                                # the window is full of tensors still to come: read directly
                    self._cv.wait(0.2)
                self._pending.discard(name)
                hit = self._staged.pop(name, None)
                if hit is not None:
                    t, ev = hit
                    self._inflight -= t.numel() * t.element_size()
                    self.stats["hits"] += 1
                    self.stats["wait_s"] += time.time() - t0
                    self._cv.notify_all()
                    if ev is not None:
                        cur = torch.cuda.current_stream(self.device)
                        cur.wait_event(ev)
                        t.record_stream(cur)                 # allocated on the worker's stream, used on this one
                    return t
            self.stats["misses"] += 1
        t = self.inner.get(name)
        self.stats["direct_bytes"] += t.numel() * t.element_size()
        return t

    def _claimed_or_near(self, name: str) -> bool:
        """True while waiting for the workers beats reading ``name`` directly: it is among the next tensors they will
        take (or one of them is reading it now)."""
        return self._idx[name] < self._next + 64

    def _drop_passed(self, name: str) -> bool:
        """Free the read-ahead window of staged tensors that sort before ``name``: the consumer went past them without
        asking (a tensor this model does not use). Called with the lock held; True if anything was freed."""
        mine = self._idx[name]
        gone = [n for n in self._staged if self._idx[n] < mine]
        for n in gone:
            t, _ = self._staged.pop(n)
            self._inflight -= t.numel() * t.element_size()
            self._pending.discard(n)
        if gone:
            self._cv.notify_all()
        return bool(gone)

    def close(self):
        with self._cv:
            self._stop = True
            self._staged.clear()
            self._cv.notify_all()
        for t in self._threads:
            t.join(timeout=5)

    def summary(self) -> dict:
        s = dict(self.stats)
        s["read_gbs_per_worker"] = round(s["bytes"] / 1e9 / s["read_s"], 2) if s["read_s"] > 0 else None
        return s


def open_checkpoint(model_dir: str, device="cpu", workers: Optional[int] = None) -> TensorSource:
    """The source a loader should build from: read-ahead workers in front of the lazy shard reader
    (``VELO_LOAD_WORKERS`` / ``workers`` = 0 gives the plain reader)."""
    n = int(os.environ.get("VELO_LOAD_WORKERS", "4")) if workers is None else workers
    src = SafetensorsSource(model_dir)
    return PrefetchSource(src, device, workers=n) if n > 0 else src


def load_report(src: TensorSource, total_s: float) -> str:
    """One ``[load]`` line splitting ``total_s`` into what the reader threads did and what the builder waited for."""
    if not isinstance(src, PrefetchSource):
        return f"[load] weights {total_s:.1f}s (no read-ahead)"
    st = src.summary()
    return (f"[load] weights {total_s:.1f}s: read {st['bytes'] / 1e9:.2f} GB by {len(src._threads)} workers "
            f"({st['read_s']:.1f} worker-s, {st['read_gbs_per_worker']} GB/s each), builder waited {st['wait_s']:.1f}s for "
            f"tensors, quantise / tile / upload of the rest {max(0.0, total_s - st['wait_s']):.1f}s; "
            f"{st['hits']} staged, {st['misses']} direct ({st['direct_bytes'] / 1e9:.2f} GB)")


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
