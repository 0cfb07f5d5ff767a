"""Single-call generation API: build or load a model on this process's GPU (one rank of a tensor-
parallel group when ``torch.distributed`` is initialised) and generate greedily. This is the thin
public entry the benchmarks and examples use; the serving path wraps the same runtime in the
continuous-batching scheduler.
"""
from __future__ import annotations

import os
import time
from typing import Callable, List, Optional, Sequence

import torch

from ..checkpoint.synthetic import SyntheticSource
from ..config import ModelConfig, preset
from ..models.runtime import GpuModel
from ..models.weights import ModelBuilder, ModelWeights


class LLM:
    def __init__(self, model: GpuModel, max_batch: int, max_seq: int):
        self.model = model
        self.cfg = model.cfg
        self.max_batch, self.max_seq = max_batch, max_seq

    # ------------------------------------------------------------ construction
    @classmethod
    def synthetic(cls, name_or_cfg="27b", recipe: str = "all", seed: int = 0, device=None, max_batch: int = 4,
                  max_seq: int = 4096, tp_rank: int = 0, tp_world: int = 1, comm=None, mtp: bool = False,
                  prefill_chunk: int = 4096) -> "LLM":
        cfg = name_or_cfg if isinstance(name_or_cfg, ModelConfig) else preset(name_or_cfg, mtp=mtp)
        device = device or f"cuda:{torch.cuda.current_device()}"
        with torch.cuda.device(device):
            w = ModelBuilder(cfg, SyntheticSource(cfg, seed, device), recipe=recipe, device=device,
                             tp_rank=tp_rank, tp_world=tp_world).build()
            return cls.from_weights(w, device, max_batch, max_seq, comm, prefill_chunk)

    @classmethod
    def from_dir(cls, model_dir: str, device=None, max_batch: int = 8, max_seq: int = 4096, recipe: str = "off",
                 tp_rank: int = 0, tp_world: int = 1, comm=None, prefill_chunk: int = 4096) -> "LLM":
        from ..checkpoint.io import open_checkpoint
        cfg = ModelConfig.from_json(os.path.join(model_dir, "config.json"))
        device = device or f"cuda:{torch.cuda.current_device()}"
        with torch.cuda.device(device):
            src = open_checkpoint(model_dir, device)
            try:
                w = ModelBuilder(cfg, src, recipe=recipe, device=device, tp_rank=tp_rank, tp_world=tp_world).build()
            finally:
                if hasattr(src, "close"):
                    src.close()
            return cls.from_weights(w, device, max_batch, max_seq, comm, prefill_chunk)

    @classmethod
    def from_weights(cls, w: ModelWeights, device, max_batch: int, max_seq: int, comm=None,
                     prefill_chunk: int = 4096) -> "LLM":
        gm = GpuModel(w, device=device, max_cols=max(16, max_batch), comm=comm, prefill_chunk=prefill_chunk)
        # lanes + 16 verify checkpoints + 1 tree scratch + one prompt checkpoint per lane
        gm.alloc_state(max_batch, max_batch + 17 + max_batch, max_seq)
        return cls(gm, max_batch, max_seq)

    # ------------------------------------------------------------ generation
    def generate(self, prompt: Sequence[int], max_new_tokens: int, slot: int = 0, use_graph: bool = True,
                 on_token: Optional[Callable[[int], None]] = None) -> List[int]:
        """Greedy generation of one sequence. Every step copies its inputs from pinned host memory and
        reads the new token back to the host, as the serving loop does."""
        gm = self.model
        assert len(prompt) + max_new_tokens <= self.max_seq
        gm.zero_slot(slot)
        logits, _ = gm.prefill(slot, list(prompt), 0, want_hidden=False)
        tok = self._argmax_global(logits.unsqueeze(0))[0]
        out = [tok]
        if on_token:
            on_token(tok)
        pos = len(prompt)
        while len(out) < max_new_tokens:
            tok = self.decode_step([tok], [pos], [slot], use_graph)[0]
            out.append(tok)
            if on_token:
                on_token(tok)
            pos += 1
        return out

    def decode_step(self, tokens, pos, slots, use_graph: bool = True) -> List[int]:
        """One greedy decode step for ``len(tokens)`` lanes; returns the new token ids on the host."""
        gm = self.model
        if use_graph:
            return gm.replay_decode(tokens, pos, slots).tolist()
        logits, _ = gm.decode(tokens, pos, slots)
        return logits.argmax(-1).tolist()

    def _argmax_global(self, logits: torch.Tensor) -> List[int]:
        return logits.argmax(-1).tolist()      # logits returned by the runtime are already full-vocabulary
