"""Tokenizer and chat template: HF ``tokenizers`` for BPE, ``jinja2`` for the model's own chat template.

Mirrors the reference wrapper (reference: src/tokenizer.rs:17-204): the template comes from
``chat_template.jinja`` or ``tokenizer_config.json``; context variables are ``messages``, ``tools``,
``add_generation_prompt``, ``enable_thinking`` and ``reasoning_effort``; the stop-token *set* is the
union of what generation_config / tokenizer_config / config declare (plus end-of-document style tokens
when the vocabulary has them); think tags are looked up in the vocabulary.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional, Sequence, Set, Tuple

import jinja2
from jinja2.sandbox import ImmutableSandboxedEnvironment
from tokenizers import Tokenizer

DEFAULT_TEMPLATE = (
    "{% for m in messages %}<|im_start|>{{ m['role'] }}\n{{ m['content'] if m['content'] is string else '' }}"
    "<|im_end|>\n{% endfor %}{% if add_generation_prompt %}<|im_start|>assistant\n"
    "{% if enable_thinking is defined and enable_thinking is false %}<think>\n\n</think>\n\n{% endif %}{% endif %}")


def _raise(msg):
    raise jinja2.TemplateError(msg)


def _tojson(x, ensure_ascii=False, indent=None, **_):
    return json.dumps(x, ensure_ascii=ensure_ascii, indent=indent)


class ChatTokenizer:
    def __init__(self, tok: Tokenizer, template: str, model_dir: Optional[str] = None, extra_cfg: Optional[dict] = None):
        self.tok = tok
        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, extensions=["jinja2.ext.loopcontrols"])
        env.filters["tojson"] = _tojson
        env.globals["raise_exception"] = _raise
        self.template = env.from_string(template)
        self.model_dir = model_dir
        self.cfg = extra_cfg or {}
        vocab = tok.get_vocab()
        self.think_open = "<think>" if "<think>" in vocab else None
        self.think_close = "</think>" if "</think>" in vocab else None
        if self.think_open is None:
            # fall back to the textual tags: splitting works on decoded text either way
            self.think_open, self.think_close = "<think>", "</think>"

    # ------------------------------------------------------------ loading
    @classmethod
    def from_dir(cls, model_dir: str, tokenizer_path: Optional[str] = None) -> "ChatTokenizer":
        path = tokenizer_path or os.path.join(model_dir, "tokenizer.json")
        tok = Tokenizer.from_file(path)
        template = None
        jpath = os.path.join(model_dir, "chat_template.jinja")
        cfg: Dict[str, Any] = {}
        tcp = os.path.join(model_dir, "tokenizer_config.json")
        if os.path.exists(tcp):
            with open(tcp) as f:
                cfg["tokenizer_config"] = json.load(f)
        if os.path.exists(jpath):
            with open(jpath) as f:
                template = f.read()
        elif "tokenizer_config" in cfg and cfg["tokenizer_config"].get("chat_template"):
            template = cfg["tokenizer_config"]["chat_template"]
            if isinstance(template, list):      # named templates: take the default
                template = next((t["template"] for t in template if t.get("name") == "default"), template[0]["template"])
        for name in ("generation_config.json", "config.json"):
            pth = os.path.join(model_dir, name)
            if os.path.exists(pth):
                with open(pth) as f:
                    cfg[name[:-5]] = json.load(f)
        return cls(tok, template or DEFAULT_TEMPLATE, model_dir, cfg)

    # ------------------------------------------------------------ basic ops
    def encode(self, text: str) -> List[int]:
        return self.tok.encode(text, add_special_tokens=False).ids

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = False) -> str:
        return self.tok.decode(list(ids), skip_special_tokens=skip_special_tokens)

    def token_id(self, s: str) -> Optional[int]:
        return self.tok.token_to_id(s)

    @property
    def vocab_size(self) -> int:
        return self.tok.get_vocab_size()

    # ------------------------------------------------------------ stop tokens
    def stop_token_ids(self) -> Set[int]:
        out: Set[int] = set()

        def add(v):
            if isinstance(v, int):
                out.add(v)
            elif isinstance(v, list):
                for x in v:
                    add(x)
            elif isinstance(v, str):
                i = self.token_id(v)
                if i is not None:
                    out.add(i)
            elif isinstance(v, dict) and "content" in v:
                add(v["content"])

        gc = self.cfg.get("generation_config", {})
        add(gc.get("eos_token_id"))
        tc = self.cfg.get("tokenizer_config", {})
        add(tc.get("eos_token"))
        c = self.cfg.get("config", {})
        for scope in (c, c.get("text_config", {})):
            add(scope.get("eos_token_id"))
            add(scope.get("eod_token_id"))
        for s in ("<|im_end|>", "<|endoftext|>", "<｜hy_EOT｜>"):
            i = self.token_id(s)
            if i is not None and (s != "<|endoftext|>" or not out):
                out.add(i)
        return out

    def think_tags(self) -> Tuple[str, str]:
        return self.think_open, self.think_close

    # ------------------------------------------------------------ chat template
    def render(self, messages: List[dict], tools: Optional[List[dict]] = None, add_generation_prompt: bool = True,
               enable_thinking: Optional[bool] = None, reasoning_effort: Optional[str] = None) -> str:
        ctx: Dict[str, Any] = {"messages": messages, "add_generation_prompt": add_generation_prompt}
        if tools:
            ctx["tools"] = tools
        if enable_thinking is not None:
            ctx["enable_thinking"] = enable_thinking
        if reasoning_effort is not None:
            ctx["reasoning_effort"] = reasoning_effort
        return self.template.render(**ctx)

    def apply_chat_template(self, messages, tools=None, enable_thinking=None, reasoning_effort=None) -> Tuple[str, List[int]]:
        text = self.render(messages, tools, True, enable_thinking, reasoning_effort)
        return text, self.encode(text)

    def checkpoint_position(self, messages, tools=None, enable_thinking=None, reasoning_effort=None,
                            full_ids: Optional[List[int]] = None) -> Optional[int]:
        """Token position of the conversation boundary: the length of the rendering *without* the
        generation prompt when it is a token-prefix of the full prompt."""
        try:
            text = self.render(messages, tools, False, enable_thinking, reasoning_effort)
        except jinja2.TemplateError:
            return None
        ids = self.encode(text)
        if full_ids is not None and full_ids[:len(ids)] != ids:
            # tokenisation merged across the boundary: back off to the longest common prefix
            n = 0
            while n < min(len(ids), len(full_ids)) and ids[n] == full_ids[n]:
                n += 1
            return n or None
        return len(ids) or None


def build_byte_tokenizer(specials: Sequence[str] = ("<|im_start|>", "<|im_end|>", "<|endoftext|>", "<think>", "</think>",
                                                     "<tool_call>", "</tool_call>")) -> Tokenizer:
    """A self-contained byte-level tokenizer (256 byte tokens + specials) for tests and synthetic models."""
    from tokenizers import AddedToken, decoders, models, pre_tokenizers
    alphabet = pre_tokenizers.ByteLevel.alphabet()
    vocab = {ch: i for i, ch in enumerate(sorted(alphabet))}
    tok = Tokenizer(models.BPE(vocab=vocab, merges=[]))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)
    tok.decoder = decoders.ByteLevel()
    tok.add_special_tokens([AddedToken(s, special=True) for s in specials])
    return tok
