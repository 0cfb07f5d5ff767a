"""Quantization recipes: which tensor group is stored in which format.

Grammar (reference: src/quant.rs:334-418): comma-separated tokens ``group[:fmt]`` or ``-group``;
``fmt`` is ``nvfp4`` (default), ``fp8`` or ``bf16``; ``all`` expands to every group. Later tokens
override earlier ones. Examples: ``all`` (nvfp4-full), ``all,gdn:fp8`` (nvfp4-mixed),
``all,-router,-embed,-lmhead``.
"""
from __future__ import annotations

from typing import Dict, Optional

GROUPS = ("mlp", "attn", "gdn", "lmhead", "embed", "mtp", "router", "expert")
NAMED_RECIPES = {"nvfp4-full": "all", "nvfp4-mixed": "all,gdn:fp8", "gdn4": "all", "bf16": "off"}


def group_of(name: str) -> str:
    """Tensor name -> group. Routing gates are tested first so ``-router`` also covers the MTP
    head's router and shared-expert gate."""
    if ".mlp.gate.weight" in name or ".shared_expert_gate." in name or ".router." in name:
        return "router"
    if name.startswith("mtp.") or ".eh_proj" in name:
        return "mtp"
    if "lm_head" in name:
        return "lmhead"
    if "embed_tokens" in name:
        return "embed"
    if ".mlp.experts." in name:
        return "expert"
    if ".mlp." in name:
        return "mlp"
    if ".self_attn." in name:
        return "attn"
    if ".linear_attn." in name and ("in_proj" in name or "out_proj" in name):
        return "gdn"
    return "other"


def parse_recipe(spec: str) -> Optional[Dict[str, str]]:
    """Recipe string -> {group: fmt}; ``None`` means no quantization at all."""
    spec = NAMED_RECIPES.get(spec.strip(), spec.strip())
    if spec in ("", "off", "none"):
        return None
    out: Dict[str, str] = {}
    for tok in (t.strip() for t in spec.split(",")):
        if not tok:
            continue
        neg = tok.startswith("-")
        if neg:
            tok = tok[1:]
        name, _, fmt = tok.partition(":")
        fmt = fmt or "nvfp4"
        if fmt not in ("nvfp4", "fp8", "bf16"):
            raise ValueError(f"unknown format {fmt!r} in recipe")
        if name == "all":
            groups = list(GROUPS)
        elif name in GROUPS:
            groups = [name]
        else:
            raise ValueError(f"unknown group {name!r} in recipe")
        for g in groups:
            out.pop(g, None)
            if not neg and fmt != "bf16":
                out[g] = fmt
    return out


def fmt_for(recipe: Optional[Dict[str, str]], name: str) -> str:
    if recipe is None:
        return "bf16"
    return recipe.get(group_of(name), "bf16")
