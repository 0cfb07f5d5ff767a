"""Tool parsing, chat template, stream splitting and the HTTP API (CPU oracle backend)."""
import json
import os

import pytest

from velogb10_b200.server import tools as T
from velogb10_b200.server.api import StreamSplitter, split_think

TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {
    "city": {"type": "string"}, "days": {"type": "integer"}, "exact": {"type": "boolean"}, "opts": {"type": "object"},
    "temp": {"type": "number"}, "tags": {"type": "array"}}}}}]


def test_tool_call_parse_and_coercion():
    out = T.parse("Let me check.\n<tool_call>\n<function=get_weather>\n<parameter=city>\nParis\n</parameter>\n"
                  "<parameter=days>\n3\n</parameter>\n<parameter=exact>\ntrue\n</parameter>\n"
                  "<parameter=opts>\n{\"a\":1}\n</parameter>\n<parameter=temp>\n2.5\n</parameter>\n"
                  "<parameter=tags>\n[1,2]\n</parameter>\n</function>\n</tool_call>", TOOLS)
    assert out.content == "Let me check." and len(out.tool_calls) == 1
    a = json.loads(out.tool_calls[0].arguments)
    assert a == {"city": "Paris", "days": 3, "exact": True, "opts": {"a": 1}, "temp": 2.5, "tags": [1, 2]}
    assert out.tool_calls[0].to_openai(0)["function"]["name"] == "get_weather"


def test_tool_call_ids_unique_truncation_and_multiline():
    two = T.parse("<tool_call>\n<function=a>\n<parameter=x>\n1\n</parameter>\n</function>\n</tool_call>\n"
                  "<tool_call>\n<function=b>\n</function>\n</tool_call>")
    assert [c.name for c in two.tool_calls] == ["a", "b"]
    again = T.parse("<tool_call>\n<function=a>\n</function>\n</tool_call>")
    ids = {c.id for c in two.tool_calls} | {again.tool_calls[0].id}
    assert len(ids) == 3
    cut = T.parse("thinking\n<tool_call>\n<function=get_weather>\n<parameter=city>\nPar", TOOLS)
    assert cut.tool_calls == [] and cut.content == "thinking"
    assert T.parse("There is no tool for that.", TOOLS).content == "There is no tool for that."
    ml = T.parse("<tool_call>\n<function=f>\n<parameter=code>\nline1\n  line2\n</parameter>\n</function>\n</tool_call>")
    assert json.loads(ml.tool_calls[0].arguments)["code"] == "line1\n  line2"
    bad = T.parse("<tool_call>\n<function=get_weather>\n<parameter=days>\nthree\n</parameter>\n</function>\n</tool_call>", TOOLS)
    assert json.loads(bad.tool_calls[0].arguments)["days"] == "three"


def test_hy3_markup():
    out = T.parse("Let me check.\n<tool_calls:opensource>\n<tool_call:opensource>get_weather<tool_sep:opensource>\n"
                  "<arg_key:opensource>city</arg_key:opensource>\n<arg_value:opensource>Paris</arg_value:opensource>\n"
                  "<arg_key:opensource>days</arg_key:opensource>\n<arg_value:opensource>3</arg_value:opensource>\n"
                  "</tool_call:opensource>\n</tool_calls:opensource>", TOOLS)
    assert out.content == "Let me check."
    assert json.loads(out.tool_calls[0].arguments) == {"city": "Paris", "days": 3}
    cut = T.parse("thinking\n<tool_call:opensource>get_weather<tool_sep:opensource>\n<arg_key:opensource>city", TOOLS)
    assert cut.tool_calls == [] and cut.content == "thinking"


def test_stream_splitter():
    full = "plan it</think>\n\nHello <tool_call>\n<function=f>\n</function>\n</tool_call>"
    sp = StreamSplitter("<think>", "</think>", True, [])
    got = []
    for i in range(1, len(full) + 1):
        got += sp.feed(full[:i])
    got += sp.feed(full, final=True)
    assert "".join(s for k, s in got if k == "reasoning") == "plan it"
    assert "".join(s for k, s in got if k == "content") == "Hello "
    assert sp.content.startswith("Hello <tool_call>") and sp.tool_hold
    assert all("<" not in s for k, s in got if k == "content")
    # a think block opening inside content, and stop strings
    sp2 = StreamSplitter("<think>", "</think>", False, ["STOP"])
    out = []
    text = "A<think>hm</think> B and STOP never"
    for i in range(1, len(text) + 1):
        out += sp2.feed(text[:i])
        if sp2.stopped:
            break
    assert sp2.stopped and "".join(s for k, s in out if k == "content") == "AB and "
    assert "".join(s for k, s in out if k == "reasoning") == "hm"
    assert split_think("x</think>  y", "<think>", "</think>", True) == ("x", "y")
    assert split_think("plain", "<think>", "</think>", False) == ("", "plain")


def test_chat_template_and_checkpoint_position():
    from velogb10_b200.server.tokenizer import ChatTokenizer, DEFAULT_TEMPLATE, build_byte_tokenizer
    tok = ChatTokenizer(build_byte_tokenizer(), DEFAULT_TEMPLATE)
    msgs = [{"role": "user", "content": "hi there"}]
    text, ids = tok.apply_chat_template(msgs)
    assert text == "<|im_start|>user\nhi there<|im_end|>\n<|im_start|>assistant\n"
    assert tok.decode(ids) == text
    ck = tok.checkpoint_position(msgs, full_ids=ids)
    assert 0 < ck < len(ids) and tok.decode(ids[:ck]).endswith("<|im_end|>\n")
    nt, _ = tok.apply_chat_template(msgs, enable_thinking=False)
    assert nt.endswith("<think>\n\n</think>\n\n")
    assert tok.token_id("<|im_end|>") in tok.stop_token_ids()
    assert tok.encode("héllo") and tok.decode(tok.encode("héllo")) == "héllo"


@pytest.fixture(scope="module")
def client():
    from fastapi.testclient import TestClient
    from velogb10_b200.checkpoint.synthetic import SyntheticSource
    from velogb10_b200.config import tiny_hybrid
    from velogb10_b200.engine.mtp import MtpPolicy
    from velogb10_b200.engine.scheduler import Scheduler
    from velogb10_b200.models.oracle import OracleModel
    from velogb10_b200.models.weights import ModelBuilder
    from velogb10_b200.server.api import AppState, EngineLoop, create_app
    from velogb10_b200.server.tokenizer import ChatTokenizer, DEFAULT_TEMPLATE, build_byte_tokenizer
    cfg = tiny_hybrid(mtp=True)
    w = ModelBuilder(cfg, SyntheticSource(cfg, 0, std=0.08), recipe="all").build()
    tok = ChatTokenizer(build_byte_tokenizer(), DEFAULT_TEMPLATE)
    sched = Scheduler(OracleModel(w), 2, 96, eos_ids=sorted(tok.stop_token_ids()), policy=MtpPolicy("on", depth=3))
    eng = EngineLoop(sched)
    eng.start()
    app = create_app(AppState(eng, tok, "tiny-test", 96, max_tokens=16, default_presence_penalty=0.0))
    with TestClient(app) as c:
        yield c
    eng.stop()


def test_http_models_and_health(client):
    assert client.get("/health").json() == {"status": "ok"}
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny-test"
    assert client.get("/v1/models/tiny-test").status_code == 200
    assert client.get("/v1/models/other").status_code == 404


def test_http_chat_blocking_stream_and_errors(client):
    body = {"model": "tiny-test", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 8, "temperature": 0,
            "seed": 7}
    r = client.post("/v1/chat/completions", json=body)
    assert r.status_code == 200
    j = r.json()
    assert j["object"] == "chat.completion" and j["id"].startswith("chatcmpl-")
    assert j["usage"]["completion_tokens"] <= 8 and j["usage"]["total_tokens"] > j["usage"]["prompt_tokens"]
    assert j["choices"][0]["finish_reason"] in ("length", "stop")
    assert {"prompt_ms", "predicted_ms", "prompt_per_second", "predicted_per_second"} <= set(j["timings"])
    text1 = j["choices"][0]["message"]["content"]
    # greedy + same prompt again (prefix cache hit) gives the same text
    assert client.post("/v1/chat/completions", json=body).json()["choices"][0]["message"]["content"] == text1
    # streaming
    with client.stream("POST", "/v1/chat/completions", json={**body, "stream": True,
                                                              "stream_options": {"include_usage": True}}) as s:
        lines = [l for l in s.iter_lines() if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    assert chunks[0]["choices"][0]["delta"] == {"role": "assistant"}
    assert chunks[-1]["choices"] == [] and "usage" in chunks[-1] and "timings" in chunks[-1]
    assert chunks[-2]["choices"][0]["finish_reason"] in ("length", "stop") and chunks[-2]["choices"][0]["delta"] == {}
    streamed = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks[:-1] if c["choices"])
    assert streamed == (text1 or "")
    # context overflow -> 400 with the OpenAI error shape
    big = {"model": "tiny-test", "messages": [{"role": "user", "content": "x" * 200}]}
    e = client.post("/v1/chat/completions", json=big)
    assert e.status_code == 400 and e.json()["error"]["code"] == "context_length_exceeded"
    # sampling path with stop list accepted as a string
    r2 = client.post("/v1/chat/completions", json={**body, "temperature": 0.8, "top_k": 5, "stop": "zzz",
                                                   "presence_penalty": 0.5, "repetition_penalty": 1.1})
    assert r2.status_code == 200


def test_cli_arg_parsing_and_scripts(tmp_path):
    from velogb10_b200 import cli
    a = cli.parse_args(["--server", "--model-dir", "/m", "--max-batch=4", "--mtp", "off", "--zero-kv"])
    assert a == {"--server": "1", "--model-dir": "/m", "--max-batch": "4", "--mtp": "off", "--zero-kv": "1"}
    assert cli.derive_model_name({"--model-dir": "/x/qwen-27b/"}) == "qwen-27b"
    assert cli.main([]) == 0
    import subprocess, sys, os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "ck")
    r = subprocess.run([sys.executable, os.path.join(root, "convert_model.py"), "--synthetic", "tiny", "--out", out],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    q = str(tmp_path / "q")
    r = subprocess.run([sys.executable, os.path.join(root, "quantize_nvfp4.py"), "--model-dir", out, "--out", q,
                        "--recipe", "all"], capture_output=True, text=True)
    assert r.returncode == 0 and json.loads(r.stdout)["nvfp4"] > 0, r.stderr
    assert os.path.exists(os.path.join(q, "tokenizer.json")) and os.path.exists(os.path.join(q, "chat_template.jinja"))
    g = subprocess.run([sys.executable, "-m", "velogb10_b200", "--generate", "--cpu", "--model-dir", q, "--prompt", "hi",
                        "--max-new", "4"], capture_output=True, text=True, cwd=root)
    assert g.returncode == 0 and len(json.loads(g.stdout)["tokens"]) == 4, g.stderr


def test_http_stop_string_that_matches_ends_both_modes(client):
    """A stop string that does occur: the handler cancels the request, the scheduler must still deliver the final
    event, and both the blocking reply and the stream (finish chunk + [DONE]) must arrive with the text cut."""
    body = {"model": "tiny-test", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 16, "temperature": 0,
            "seed": 7}
    full = client.post("/v1/chat/completions", json=body).json()["choices"][0]["message"]["content"] or ""
    assert len(full) >= 3, full
    i = next(k for k in range(1, len(full)) if full[k] not in full[:k])
    stop = full[i]
    r = client.post("/v1/chat/completions", json={**body, "stop": [stop]})
    assert r.status_code == 200
    j = r.json()
    assert (j["choices"][0]["message"]["content"] or "") == full[:i] and j["choices"][0]["finish_reason"] == "stop"
    with client.stream("POST", "/v1/chat/completions", json={**body, "stop": stop, "stream": True}) as s:
        lines = [l for l in s.iter_lines() if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    assert chunks[-1]["choices"][0]["finish_reason"] == "stop"
    assert "".join(c["choices"][0]["delta"].get("content", "") for c in chunks if c["choices"]) == full[:i]


def test_prompt_and_raw_output_dumps(client, monkeypatch, tmp_path, capsys):
    """VELO_DUMP_PROMPT writes the rendered prompt of each request to a numbered file; with tools offered and no call
    parsed the raw model output is logged even without VELO_DUMP_TOOLS."""
    import tempfile
    monkeypatch.setenv("VELO_DUMP_PROMPT", "1")
    monkeypatch.setattr(tempfile, "tempdir", str(tmp_path))
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object", "properties": {}}}}]
    body = {"model": "tiny-test", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "temperature": 0,
            "tools": tools}
    assert client.post("/v1/chat/completions", json=body).status_code == 200
    files = sorted(os.listdir(tmp_path))
    assert files and files[0].startswith("velo_prompt_") and "hi" in open(os.path.join(tmp_path, files[0])).read()
    err = capsys.readouterr().err
    assert "[req] dumped prompt" in err and "[req] raw model output" in err
