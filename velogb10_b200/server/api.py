"""OpenAI-compatible HTTP API: ``POST /v1/chat/completions`` (streaming SSE and blocking),
``GET /v1/models``, ``GET /v1/models/{id}``, ``GET /health``, permissive CORS.

Field set and streaming behaviour follow the reference server (reference: src/server.rs:119-183 request,
:185-255 response/timings, :263-636 handler, :637-649 router): sampling defaults temperature 0.7 /
top_p 0.8 / top_k 20, ``stop`` as string or list, seeds, penalties with server-side defaults,
``reasoning_content`` split on the think tags, tool-call hold-back with one final ``tool_calls`` delta,
``stream_options.include_usage``, llama.cpp-style ``timings``, a 400 JSON error when the prompt does not
fit the context, and ``data: [DONE]``.

The scheduler runs on its own thread (``EngineLoop``); HTTP handlers talk to it through a thread-safe
inbox and receive token events on asyncio queues.
"""
from __future__ import annotations

import asyncio
import itertools
import json
import os
import queue
import sys
import tempfile
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, AsyncIterator, Dict, List, Optional, Tuple

from fastapi import FastAPI
from fastapi import Request as HttpRequest
from fastapi.middleware.cors import CORSMiddleware
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from ..engine.sampling import SamplingParams
from ..engine.scheduler import Request, Scheduler
from . import tools as T
from .tokenizer import ChatTokenizer


# ------------------------------------------------------------------ engine thread

class EngineLoop:
    """Owns the scheduler: admits requests from the inbox, steps while there is work, blocks when idle.
    If the scheduler raises, the loop records the error and fails every pending request instead of
    leaving clients hanging (the reference exits the process; embedding hosts can check ``error``)."""

    def __init__(self, scheduler: Scheduler, lockstep=None):
        self.s = scheduler
        self.lockstep = lockstep          # parallel.lockstep.Lockstep on the head rank of a multi-process TP group
        self.inbox: "queue.Queue[Optional[Request]]" = queue.Queue()
        self.thread = threading.Thread(target=self._run, daemon=True, name="engine-loop")
        self.error: Optional[BaseException] = None
        self.running = False

    def start(self):
        self.running = True
        self.thread.start()

    def stop(self):
        self.running = False
        self.inbox.put(None)
        self.thread.join(timeout=10)

    def submit(self, req: Request):
        if self.error is not None:
            raise RuntimeError(f"engine stopped: {self.error}")
        self.inbox.put(req)

    def _drain(self, block: bool):
        try:
            item = self.inbox.get(block=block, timeout=0.5 if block else None)
            while True:
                if item is not None:
                    self.s.submit(item)
                item = self.inbox.get_nowait()
        except queue.Empty:
            pass

    def _run_lockstep(self):
        """Head loop of a tensor-parallel group: ship each step's admissions and cancellations to the
        mirror ranks before acting on them."""
        while self.running:
            admits = []
            try:
                item = self.inbox.get(block=self.s.idle(), timeout=0.5)
                while True:
                    if item is not None:
                        admits.append(item)
                    item = self.inbox.get_nowait()
            except queue.Empty:
                pass
            # one snapshot of the owners' flags per step, queued requests included; the scheduler on every rank
            # acts on exactly this list (a flag that flips after this line belongs to the next step)
            cancels = self.s.pending_cancels()
            if admits or not self.s.idle():
                self.lockstep.head_step(admits, cancels)
        self.lockstep.head_step([], [], stop=True)

    def _run(self):
        try:
            if self.lockstep is not None:
                self._run_lockstep()
                return
            while self.running:
                self._drain(block=self.s.idle())
                if not self.s.idle():
                    self.s.step()
        except BaseException as e:  # noqa: BLE001 - reported to every waiter
            self.error = e
            for lane in list(self.s.lanes):
                if lane.req.on_finish:
                    lane.req.on_finish("error", {})
            for req in list(self.s.queue):
                if req.on_finish:
                    req.on_finish("error", {})
            raise


# ------------------------------------------------------------------ text splitting

class StreamSplitter:
    """Turns the growing decoded text into deltas: reasoning before the think-close tag, content after
    (leading whitespace after the tag dropped), content held back from the first ``<tool_call`` or any
    tail that could still become one, stop strings cutting the text."""

    TOOL_PREFIX = "<tool_call"

    def __init__(self, think_open: str, think_close: str, start_in_think: bool, stop: List[str]):
        self.open, self.close = think_open, think_close
        self.in_think = start_in_think
        self.stop = [s for s in stop if s]
        self.text = ""
        self.emitted = 0            # characters of self.text already classified
        self.reasoning = ""
        self.content = ""
        self.tool_hold = False
        self.stopped = False
        self.strip_next = False

    @staticmethod
    def _partial_tail(s: str, tag: str) -> int:
        """Length of the longest proper prefix of ``tag`` that ends ``s``."""
        for n in range(min(len(tag) - 1, len(s)), 0, -1):
            if s.endswith(tag[:n]):
                return n
        return 0

    def feed(self, full_text: str, final: bool = False) -> List[Tuple[str, str]]:
        """``full_text`` is everything decoded so far. Returns [(kind, delta)] with kind in
        reasoning / content."""
        out: List[Tuple[str, str]] = []
        if self.stopped:
            return out
        self.text = full_text
        for s in self.stop:
            i = self.text.find(s, max(0, self.emitted - len(s)))
            if i >= 0:
                self.text = self.text[:i]
                self.stopped = True
                final = True
                break
        while self.emitted < len(self.text):
            rest = self.text[self.emitted:]
            if self.in_think:
                i = rest.find(self.close)
                if i >= 0:
                    seg = rest[:i]
                    self.emitted += i + len(self.close)
                    self.in_think = False
                    self.strip_next = True
                else:
                    hold = 0 if final else max(self._partial_tail(rest, self.close),
                                               max((self._partial_tail(rest, s) for s in self.stop), default=0))
                    seg = rest[:len(rest) - hold]
                    self.emitted += len(seg)
                if seg:
                    self.reasoning += seg
                    out.append(("reasoning", seg))
                if i < 0:
                    break
            else:
                if self.strip_next:
                    stripped = rest.lstrip()
                    if not stripped and not final:
                        break
                    self.emitted += len(rest) - len(stripped)
                    rest = stripped
                    self.strip_next = False
                    if not rest:
                        break
                if self.tool_hold:
                    self.content += rest
                    self.emitted += len(rest)
                    break
                j = rest.find(self.open) if self.open else -1
                k = rest.find(self.TOOL_PREFIX)
                cut = min([x for x in (j, k) if x >= 0], default=-1)
                if cut >= 0:
                    seg = rest[:cut]
                    if seg:
                        self.content += seg
                        out.append(("content", seg))
                    self.emitted += cut
                    if cut == j and (k < 0 or j < k):
                        self.emitted += len(self.open)
                        self.in_think = True
                    else:
                        self.tool_hold = True
                    continue
                hold = 0
                if not final:
                    hold = max(self._partial_tail(rest, self.TOOL_PREFIX), self._partial_tail(rest, self.open) if self.open else 0,
                               max((self._partial_tail(rest, s) for s in self.stop), default=0))
                seg = rest[:len(rest) - hold]
                if seg:
                    self.content += seg
                    out.append(("content", seg))
                self.emitted += len(seg)
                break
        return out


def split_think(text: str, think_open: str, think_close: str, start_in_think: bool) -> Tuple[str, str]:
    """(reasoning, content) of a finished generation."""
    sp = StreamSplitter(think_open, think_close, start_in_think, [])
    sp.feed(text, final=True)
    return sp.reasoning.strip(), sp.content


# ------------------------------------------------------------------ app state / helpers

@dataclass
class AppState:
    engine: EngineLoop
    tokenizer: ChatTokenizer
    model_name: str
    max_seq_len: int
    max_tokens: int = 8192
    default_repetition_penalty: float = 1.0
    default_presence_penalty: float = 1.5
    default_frequency_penalty: float = 0.0
    default_reasoning_effort: Optional[str] = None
    created: int = field(default_factory=lambda: int(time.time()))


def normalize_effort(v: Optional[str]) -> Optional[str]:
    if v is None:
        return None
    v = str(v).lower()
    if v in ("none", "no_think", "off", "disabled", "minimal"):
        return "no_think"
    if v in ("low",):
        return "low"
    return "high"


def timings(usage: dict) -> dict:
    t0, t1, t2 = usage.get("t_submit", 0.0), usage.get("t_first", 0.0), usage.get("t_done", 0.0)
    pm = max(1e-6, (t1 - t0) * 1e3)
    gm = max(1e-6, (t2 - t1) * 1e3)
    pn = max(0, usage.get("prompt_tokens", 0) - usage.get("prefix_hit", 0))
    gn = usage.get("completion_tokens", 0)
    return {"prompt_n": pn, "prompt_ms": pm, "prompt_per_second": pn / (pm / 1e3),
            "predicted_n": gn, "predicted_ms": gm, "predicted_per_second": gn / (gm / 1e3)}


def context_error(prompt_len: int, max_seq: int) -> dict:
    return {"error": {"message": f"This model's maximum context length is {max_seq} tokens, but the prompt has "
                                 f"{prompt_len} tokens.", "type": "invalid_request_error",
                      "code": "context_length_exceeded"}}


def map_finish(reason: str) -> str:
    return "length" if reason in ("context_length_exceeded", "length") else ("stop" if reason in ("stop", "cancelled") else reason)


# ------------------------------------------------------------------ the app

def create_app(state: AppState):
    app = FastAPI(title="velogb10_b200")
    app.add_middleware(CORSMiddleware, allow_origins=["*"], allow_methods=["*"], allow_headers=["*"])

    dump_counter = itertools.count()

    def dump_prompt(prompt_text: str):
        """VELO_DUMP_PROMPT=1: the exact rendered prompt of every request goes to a numbered file under the
        temporary directory, so the bytes a model sees can be inspected or diffed across turns
        (reference: src/server.rs:299-309)."""
        if os.environ.get("VELO_DUMP_PROMPT"):
            path = os.path.join(tempfile.gettempdir(), f"velo_prompt_{next(dump_counter)}.txt")
            try:
                with open(path, "w", encoding="utf-8") as f:
                    f.write(prompt_text)
                print(f"[req] dumped prompt ({len(prompt_text)} chars) -> {path}", file=sys.stderr, flush=True)
            except OSError:
                pass

    def log_raw_output(content: str, tools, parsed):
        """With tools offered, the model's literal output is what settles a "the tool ran but nothing happened"
        report: logged on request (VELO_DUMP_TOOLS=1) and always when tools were offered and no call was parsed
        (the model declined, or emitted a call the parser did not understand) (reference: src/server.rs:509-516,
        :587-599)."""
        if tools and (os.environ.get("VELO_DUMP_TOOLS") or not (parsed and parsed.tool_calls)):
            print(f"[req] raw model output ({len(content)} chars): {content[:1200]!r}", file=sys.stderr, flush=True)

    @app.get("/health")
    async def health():
        return {"status": "ok"}

    def model_card():
        return {"id": state.model_name, "object": "model", "created": state.created, "owned_by": "velogb10_b200"}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [model_card()]}

    @app.get("/v1/models/{model_id:path}")
    async def model(model_id: str):
        if model_id != state.model_name:
            return JSONResponse({"error": {"message": f"model {model_id!r} not found", "type": "invalid_request_error",
                                           "code": "model_not_found"}}, status_code=404)
        return model_card()

    @app.post("/v1/chat/completions")
    async def chat(http: HttpRequest):
        body = await http.json()
        tok = state.tokenizer
        messages = body.get("messages") or []
        tools = body.get("tools")
        effort = normalize_effort(body.get("reasoning_effort", state.default_reasoning_effort))
        enable_thinking = None if effort is None else effort != "no_think"
        try:
            prompt_text, ids = tok.apply_chat_template(messages, tools, enable_thinking, effort)
        except Exception as e:  # noqa: BLE001 - template failure is a 500 text body
            return PlainTextResponse(f"chat template error: {e}", status_code=500)
        dump_prompt(prompt_text)
        if len(ids) >= state.max_seq_len:
            return JSONResponse(context_error(len(ids), state.max_seq_len), status_code=400)
        ckpt_at = tok.checkpoint_position(messages, tools, enable_thinking, effort, ids)
        max_tokens = int(body.get("max_tokens") or body.get("max_completion_tokens") or state.max_tokens)
        max_tokens = max(1, min(max_tokens, state.max_tokens, state.max_seq_len - len(ids)))
        stop = body.get("stop") or []
        if isinstance(stop, str):
            stop = [stop]
        sp = SamplingParams(
            temperature=float(body.get("temperature", 0.7)), top_p=max(0.01, float(body.get("top_p", 0.8))),
            top_k=int(body.get("top_k", 20)),
            repetition_penalty=float(body.get("repetition_penalty", state.default_repetition_penalty)),
            presence_penalty=float(body.get("presence_penalty", state.default_presence_penalty)),
            frequency_penalty=float(body.get("frequency_penalty", state.default_frequency_penalty)),
            seed=body.get("seed"))
        stream = bool(body.get("stream", False))
        include_usage = bool((body.get("stream_options") or {}).get("include_usage", False))
        think_open, think_close = tok.think_tags()
        start_in_think = prompt_text.rstrip().endswith(think_open)
        loop = asyncio.get_running_loop()
        events: "asyncio.Queue[Tuple[str, Any]]" = asyncio.Queue()
        req = Request(ids, max_tokens, sp, stop_ids=tok.stop_token_ids(), ckpt_at=ckpt_at,
                      on_token=lambda t: loop.call_soon_threadsafe(events.put_nowait, ("tok", t)),
                      on_finish=lambda r, u: loop.call_soon_threadsafe(events.put_nowait, ("fin", (r, u))))
        try:
            state.engine.submit(req)
        except RuntimeError as e:
            return PlainTextResponse(str(e), status_code=503)
        cid = f"chatcmpl-{uuid.uuid4()}"
        created = int(time.time())

        def chunk(delta: dict, finish: Optional[str] = None) -> str:
            return "data: " + json.dumps({"id": cid, "object": "chat.completion.chunk", "created": created,
                                          "model": state.model_name,
                                          "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}) + "\n\n"

        async def gen_tokens() -> AsyncIterator[Tuple[str, Any]]:
            while True:
                kind, val = await events.get()
                yield kind, val
                if kind == "fin":
                    return

        if stream:
            async def sse():
                splitter = StreamSplitter(think_open, think_close, start_in_think, stop)
                out_ids: List[int] = []
                usage: dict = {}
                reason = "stop"
                yield chunk({"role": "assistant"})
                try:
                    async for kind, val in gen_tokens():
                        if kind == "tok":
                            out_ids.append(val)
                            text = tok.decode(out_ids)
                            if text.endswith("�"):
                                continue
                            for k, seg in splitter.feed(text):
                                yield chunk({"reasoning_content": seg} if k == "reasoning" else {"content": seg})
                            if splitter.stopped:
                                req.cancelled = True
                                reason = "stop"
                        else:
                            r, usage = val
                            if not splitter.stopped:
                                reason = map_finish(r)
                    for k, seg in splitter.feed(tok.decode(out_ids), final=True):
                        yield chunk({"reasoning_content": seg} if k == "reasoning" else {"content": seg})
                    if splitter.stopped:          # also when the match only completed in the final flush
                        reason = "stop"
                    parsed = T.parse(splitter.content, tools) if T.has_tool_call(splitter.content) else None
                    log_raw_output(splitter.content, tools, parsed)
                    if parsed and parsed.tool_calls:
                        yield chunk({"tool_calls": [c.to_openai(i) for i, c in enumerate(parsed.tool_calls)]})
                        reason = "tool_calls"
                    yield chunk({}, reason)
                    if include_usage:
                        u = {"prompt_tokens": usage.get("prompt_tokens", len(ids)),
                             "completion_tokens": usage.get("completion_tokens", len(out_ids))}
                        u["total_tokens"] = u["prompt_tokens"] + u["completion_tokens"]
                        yield "data: " + json.dumps({"id": cid, "object": "chat.completion.chunk", "created": created,
                                                     "model": state.model_name, "choices": [], "usage": u,
                                                     "timings": timings(usage)}) + "\n\n"
                    yield "data: [DONE]\n\n"
                finally:
                    req.cancelled = True        # a dropped connection frees the lane
            return StreamingResponse(sse(), media_type="text/event-stream")

        # ---- blocking
        out_ids = []
        usage, reason = {}, "stop"
        stopped_text: Optional[str] = None
        async for kind, val in gen_tokens():
            if kind == "tok":
                out_ids.append(val)
                if stop and len(out_ids) % 4 == 0:       # live check over the recent tail
                    tail = tok.decode(out_ids[-96:])
                    if any(s in tail for s in stop):
                        req.cancelled = True
            else:
                r, usage = val
                reason = map_finish(r)
        text = tok.decode(out_ids)
        for s in stop:
            i = text.find(s)
            if i >= 0:
                text = text[:i]
                reason = "stop"
        reasoning, content = split_think(text, think_open, think_close, start_in_think)
        parsed = T.parse(content, tools)
        log_raw_output(content, tools, parsed)
        msg: Dict[str, Any] = {"role": "assistant", "content": parsed.content or None}
        if reasoning:
            msg["reasoning_content"] = reasoning
        if parsed.tool_calls:
            msg["tool_calls"] = [c.to_openai() for c in parsed.tool_calls]
            reason = "tool_calls"
        u = {"prompt_tokens": usage.get("prompt_tokens", len(ids)), "completion_tokens": len(out_ids)}
        u["total_tokens"] = u["prompt_tokens"] + u["completion_tokens"]
        usage.setdefault("completion_tokens", len(out_ids))
        usage.setdefault("t_done", time.time())
        return {"id": cid, "object": "chat.completion", "created": created, "model": state.model_name,
                "choices": [{"index": 0, "message": msg, "finish_reason": reason}], "usage": u,
                "timings": timings(usage)}

    return app
