"""Black-box API checks against a live server on the CPU oracle path (tiny random model): OpenAI and Anthropic
endpoints, streaming, usage with cached tokens, errors, monitor and metrics routes."""
import http.client
import json
import os

import pytest
import torch

from volta_engine_b200.loader.chat_template import ChatTemplate
from volta_engine_b200.models.dense import DenseConfig, DenseModel
from volta_engine_b200.runtime.engine import Engine
from volta_engine_b200.runtime.generator import Generator
from volta_engine_b200.runtime.kv_cache import PagedKVCache
from volta_engine_b200.runtime.options import Options
from volta_engine_b200.runtime.prefix_cache import PrefixCache
from volta_engine_b200.server.app import VoltaServer
from test_tokenizer import _train


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    from volta_engine_b200.loader.tokenizer import Tokenizer
    d = str(tmp_path_factory.mktemp("tok"))
    _train(d)
    tok = Tokenizer.load(d)
    cfg = DenseConfig.tiny(vocab=512)
    model = DenseModel(cfg, "cpu").init_random(seed=0)
    kv = PagedKVCache(cfg.n_layers, model.nkv, cfg.head_dim, 64, 4, 1024, "cpu")
    eng = Engine(model, kv, use_graphs=False, prefill_chunk=64)
    opt = Options.resolve({"max_slots": 4, "prefix_interval": 64}, env={})
    gen = Generator(eng, tok, opt, prefix_cache=PrefixCache(64 << 20), eos_ids=[tok.piece_id("<|im_end|>")])
    srv = VoltaServer(gen, tok, ChatTemplate.load(d), model_name="tiny-test", api_key="sekret", max_context=1024,
                      default_max_tokens=16).start()
    yield srv
    srv.stop()


def call(srv, method, path, body=None, key="sekret", raw=False):
    c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=60)
    h = {"Content-Type": "application/json"}
    if key:
        h["Authorization"] = "Bearer " + key
    c.request(method, path, body=json.dumps(body) if body is not None and not raw else body, headers=h)
    r = c.getresponse()
    data = r.read().decode("utf-8")
    c.close()
    return r.status, data


def sse_events(data):
    out = []
    for block in data.split("\n\n"):
        ev = {}
        for ln in block.split("\n"):
            if ln.startswith("data: "):
                ev["data"] = ln[6:]
            elif ln.startswith("event: "):
                ev["event"] = ln[7:]
        if ev:
            out.append(ev)
    return out


MSG = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "Hello world! It's 2024"}]


def test_health_models_auth_and_404(server):
    assert call(server, "GET", "/health", key=None)[0] == 200
    st, body = call(server, "GET", "/v1/models")
    assert st == 200 and json.loads(body)["data"][0]["id"] == "tiny-test"
    assert call(server, "GET", "/v1/models", key="wrong")[0] == 401
    assert call(server, "GET", "/nope")[0] == 404


def test_openai_complete_and_stream_agree(server):
    st, body = call(server, "POST", "/v1/chat/completions", {"messages": MSG, "max_tokens": 12})
    assert st == 200
    full = json.loads(body)
    assert full["object"] == "chat.completion" and full["usage"]["completion_tokens"] <= 12
    text = full["choices"][0]["message"]["content"]
    st, data = call(server, "POST", "/v1/chat/completions", {"messages": MSG, "max_tokens": 12, "stream": True})
    ev = sse_events(data)
    assert ev[-1]["data"] == "[DONE]"
    chunks = [json.loads(e["data"]) for e in ev[:-1]]
    streamed = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks if c["choices"])
    assert streamed == text
    usage = [c for c in chunks if c.get("usage")][-1]["usage"]
    assert usage["prompt_tokens"] == full["usage"]["prompt_tokens"]
    assert usage["prompt_tokens_details"]["cached_tokens"] >= 0
    assert any(c["choices"] and c["choices"][0]["finish_reason"] for c in chunks)


def test_anthropic_stream_and_count_tokens(server):
    body = {"model": "x", "max_tokens": 10, "system": "Be brief.", "stream": True,
            "messages": [{"role": "user", "content": [{"type": "text", "text": "Hello world!"}]}]}
    st, data = call(server, "POST", "/v1/messages", body)
    assert st == 200
    names = [e["event"] for e in sse_events(data)]
    assert names[0] == "message_start" and names[-1] == "message_stop" and "message_delta" in names
    body["stream"] = False
    st, data = call(server, "POST", "/v1/messages", body)
    msg = json.loads(data)
    assert msg["type"] == "message" and msg["stop_reason"] in ("max_tokens", "end_turn")
    assert msg["usage"]["output_tokens"] <= 10
    st, data = call(server, "POST", "/v1/messages/count_tokens", {"messages": [{"role": "user", "content": "Hello world!"}]})
    assert st == 200 and json.loads(data)["input_tokens"] > 3


def test_errors(server):
    assert call(server, "POST", "/v1/chat/completions", "{not json", raw=True)[0] == 400
    assert call(server, "POST", "/v1/chat/completions", {"messages": []})[0] == 400
    assert call(server, "POST", "/v1/chat/completions", {"messages": MSG, "temperature": "hot"})[0] == 400
    assert call(server, "POST", "/v1/messages", {"messages": MSG[1:]})[0] == 400       # max_tokens missing
    long = [{"role": "user", "content": "word " * 3000}]
    st, data = call(server, "POST", "/v1/chat/completions", {"messages": long})
    assert st == 400 and "context" in data


def test_sampling_seed_and_stop(server):
    b = {"messages": MSG, "max_tokens": 10, "temperature": 0.8, "top_p": 0.9, "seed": 11}
    a1 = json.loads(call(server, "POST", "/v1/chat/completions", b)[1])["choices"][0]["message"]["content"]
    a2 = json.loads(call(server, "POST", "/v1/chat/completions", b)[1])["choices"][0]["message"]["content"]
    assert a1 == a2
    lp = json.loads(call(server, "POST", "/v1/chat/completions", dict(b, logprobs=True, top_logprobs=3))[1])
    assert lp["choices"][0]["logprobs"]["content"][0]["logprob"] <= 0


def test_monitor_stats_metrics(server):
    st, data = call(server, "GET", "/api/stats", key=None)
    s = json.loads(data)
    for k in ("server", "totals", "averages", "latency", "speculation", "slots", "recent", "history", "gpus", "host",
              "prefix_cache"):
        assert k in s
    assert s["totals"]["completed"] >= 1 and s["prefix_cache"]["lookups"] >= 1
    assert "<html>" in call(server, "GET", "/monitor", key=None)[1]
    prom = call(server, "GET", "/metrics/prometheus", key=None)[1]
    assert "volta_requests_total" in prom and "volta_prefix_cache_hits_total" in prom
    assert call(server, "GET", "/metrics", key=None)[0] == 200


def test_image_parts_reach_the_multimodal_front_end(server):
    import base64
    from volta_engine_b200.runtime.multimodal import MmLayout
    from volta_engine_b200.server.protocol import IMAGE_MARK, parse_anthropic, parse_openai
    png = base64.b64encode(b"\x89PNG fake").decode()
    body = {"model": "tiny-test", "max_tokens": 4, "messages": [{"role": "user", "content": [
        {"type": "text", "text": "what is "}, {"type": "image_url", "image_url": {"url": "data:image/png;base64," + png}},
        {"type": "text", "text": " ?"}]}]}
    cr = parse_openai(body, {})
    assert cr.images == [b"\x89PNG fake"] and cr.messages[0]["content"] == "what is " + IMAGE_MARK + " ?"
    ab = {"model": "m", "max_tokens": 4, "messages": [{"role": "user", "content": [
        {"type": "image", "source": {"type": "base64", "media_type": "image/png", "data": png}}, {"type": "text", "text": "hi"}]}]}
    ca = parse_anthropic(ab, {})
    assert ca.images == [b"\x89PNG fake"] and ca.messages[0]["content"].startswith(IMAGE_MARK)
    # without a vision tower the request is refused; with a front end the image bytes arrive there
    st, data = call(server, "POST", "/v1/chat/completions", body)
    assert st == 400 and "vision tower" in data
    seen = []

    class Front:
        def prepare(self, ids, images):
            seen.append(list(images))
            return ids, MmLayout(len(ids), []), None
    server.gen.mm_frontend = Front()
    try:
        st, data = call(server, "POST", "/v1/chat/completions", body)
        assert st == 200 and seen == [[b"\x89PNG fake"]] and json.loads(data)["usage"]["completion_tokens"] > 0
        bad = json.loads(json.dumps(body))
        bad["messages"][0]["content"][1]["image_url"]["url"] = "http://example.com/x.png"
        st, data = call(server, "POST", "/v1/chat/completions", bad)
        assert st == 400 and "data: URL" in data
    finally:
        server.gen.mm_frontend = None
