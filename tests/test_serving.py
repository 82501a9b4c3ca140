"""Serving shell (cider_b200/serving.py) on the CPU: the w8a8 switch, the per-request
feature cache, message parsing, parameter merging, the single-worker queue and the
HTTP layer (driven as a bare ASGI application: no HTTP client library is needed).

Behaviour checked against vlm_service/server.py:133-180 (contexts), :264-339 (result
dicts), :382-466 (messages, parameters), :469-576 (endpoint) and
vlm_service/core_infer.py:129-157 (w8a8 auto / on / off)."""
import asyncio
import base64
import json
import threading
import time

import pytest
import torch

from cider_b200 import serving
from cider_b200.serving import (BadRequest, InferenceRequest, InferenceService, RequestContextStore, SamplingDefaults,
                                SUCCESS, decode_image, merge_params, parse_messages, resolve_w8a8)

PNG = base64.b64encode(b"\x89PNG\r\n\x1a\n" + bytes(range(40))).decode()


# ----------------------------------------------------------------- w8a8: auto / on / off
def test_w8a8_off_never_converts():
    calls = []
    assert resolve_w8a8("off", lambda: True, lambda: calls.append(1)) == (False, None)
    assert calls == []


def test_w8a8_auto_follows_the_device():
    assert resolve_w8a8("auto", lambda: False, lambda: pytest.fail("must not convert")) == (False, None)
    assert resolve_w8a8("auto", lambda: True, lambda: {"converted": 7}) == (True, {"converted": 7})


def test_w8a8_auto_survives_a_failing_conversion_and_on_does_not():
    def boom():
        raise RuntimeError("no kernel library")
    assert resolve_w8a8("auto", lambda: True, boom) == (False, None)
    with pytest.raises(RuntimeError, match="no kernel library"):
        resolve_w8a8("on", lambda: True, boom)
    with pytest.raises(RuntimeError, match="not available"):
        resolve_w8a8("on", lambda: False, lambda: None)
    with pytest.raises(ValueError):
        resolve_w8a8("maybe", lambda: True, lambda: None)


# ----------------------------------------------------------------- request contexts
def test_contexts_are_per_request_id_and_expire_after_ttl():
    now = [1000.0]
    store = RequestContextStore(ttl=60, clock=lambda: now[0])
    a = store.get_or_create("a")
    assert store.get_or_create("a") is a and store.get_or_create("b") is not a
    feats, stack = a.buffers(store.now())
    feats.append("f0")
    assert store.get_or_create("a").buffers(store.now())[0] == ["f0"]  # the same lists come back
    now[0] += 59
    store.get_or_create("b").buffers(store.now())  # b is used again, a is not
    now[0] += 2
    assert store.cleanup() == 1 and len(store) == 1
    assert store.get_or_create("a").buffers(store.now())[0] == []  # a fresh context


# ----------------------------------------------------------------- messages, images, parameters
def test_parse_messages_text_and_multimodal():
    msgs = [{"role": "system", "content": "be brief"},
            {"role": "user", "content": [{"type": "text", "text": "what is "},
                                         {"type": "image_url", "image_url": {"url": "data:image/png;base64," + PNG}},
                                         {"type": "text", "text": "?"}]},
            {"role": "assistant", "content": 42}]
    parsed, images = parse_messages(msgs, external_images=[b"first"])
    assert parsed == [{"role": "system", "content": "be brief"}, {"role": "user", "content": "what is <image>?"},
                      {"role": "assistant", "content": "42"}]
    assert images[0] == b"first" and images[1].startswith(b"\x89PNG") and len(images) == 2


def test_decode_image_forms_and_errors():
    raw = base64.b64decode(PNG)
    assert decode_image(PNG) == raw and decode_image("data:image/png;base64," + PNG) == raw
    with pytest.raises(BadRequest, match="failed to decode"):
        decode_image("not base64 !!")
    with pytest.raises(BadRequest, match="invalid image data type"):
        decode_image({"url": "x"})
    with pytest.raises(BadRequest, match="not enabled"):
        decode_image("https://example.invalid/a.png")
    assert decode_image("https://example.invalid/a.png", fetch=lambda url: b"bytes of " + url.encode()) \
        == b"bytes of https://example.invalid/a.png"


def test_request_parameters_win_over_defaults():
    d = SamplingDefaults(temperature=0.7, top_k=20, top_p=0.9, repetition_penalty=1.1, max_new_tokens=100)
    assert merge_params({}, d) == {"temperature": 0.7, "topp": 0.9, "topk": 20, "repetition_penalty": 1.1,
                                   "max_new_tokens": 100, "stream": False}
    got = merge_params({"temperature": 0.0, "top_p": None, "top_k": 5, "stream": True, "max_tokens": 8}, d)
    assert got == {"temperature": 0.0, "topp": 0.9, "topk": 5, "repetition_penalty": 1.1, "max_new_tokens": 8,
                   "stream": True}


# ----------------------------------------------------------------- the worker
class FakeEngine:
    """Records what it is asked and on which thread; echoes the last user message."""

    def __init__(self):
        self.thread = threading.current_thread().name
        self.calls = []
        self.running = 0
        self.max_running = 0
        self.lock = threading.Lock()

    def _enter(self, messages, images, feats, stack):
        with self.lock:
            self.running += 1
            self.max_running = max(self.max_running, self.running)
        while len(feats) < len(images):  # "vision tower": one call per image not seen before
            feats.append(("feat", images[len(feats)]))
            stack.append(None)
        self.calls.append((threading.current_thread().name, messages[-1]["content"], len(images), len(feats)))

    def _leave(self):
        with self.lock:
            self.running -= 1

    def complete(self, messages, images, feats, stack, **params):
        self._enter(messages, images, feats, stack)
        try:
            time.sleep(0.01)
            text = messages[-1]["content"]
            if text == "fail":
                return "model_error", "", {"prefill_time": 0.5, "decode_tps": 0.0}
            if text == "raise":
                raise RuntimeError("kernel fault")
            return SUCCESS, "echo:" + text, {"prefill_time": 0.25, "decode_tps": 100.0}
        finally:
            self._leave()

    def complete_stream(self, messages, images, feats, stack, **params):
        self._enter(messages, images, feats, stack)
        try:
            timing = {"prefill_time": 0.25, "decode_tps": 50.0}
            text = messages[-1]["content"]
            if text == "fail":
                yield "model_error", "", timing
                return
            for piece in ("ec", "ho:", text):
                yield SUCCESS, piece, timing
        finally:
            self._leave()


def _service():
    svc = InferenceService(FakeEngine, ttl=60, cleanup_every=3600)
    assert svc.ready.wait(5) and svc.failed is None
    return svc


def _req(text, rid="r", stream=False, images=()):
    return InferenceRequest(rid, [{"role": "user", "content": text}], list(images), {"stream": stream})


def test_engine_lives_in_the_worker_thread_and_requests_run_one_at_a_time_in_order():
    svc = _service()
    try:
        assert svc.engine.thread == "cider-worker"
        queues = [svc.submit(_req(f"m{i}", rid=f"r{i}")) for i in range(8)]
        results = [q.get(timeout=5) for q in queues]
        assert [r["text"] for r in results] == [f"echo:m{i}" for i in range(8)]
        assert all(r["status"] == SUCCESS and r["prefill_time"] == 0.25 and r["decode_tps"] == 100.0 for r in results)
        assert [c[1] for c in svc.engine.calls] == [f"m{i}" for i in range(8)]  # arrival order
        assert {c[0] for c in svc.engine.calls} == {"cider-worker"} and svc.engine.max_running == 1
    finally:
        svc.shutdown()


def test_errors_come_back_as_results_and_the_worker_goes_on():
    svc = _service()
    try:
        bad = svc.submit(_req("fail")).get(timeout=5)
        assert bad["status"] == "model_error" and bad["error"] == "model_error" and bad["text"] == ""
        boom = svc.submit(_req("raise")).get(timeout=5)
        assert "kernel fault" in boom["status"] and boom["done"] is True
        assert svc.submit(_req("still alive")).get(timeout=5)["text"] == "echo:still alive"
    finally:
        svc.shutdown()


def test_stream_results_are_pieces_then_a_final_record():
    svc = _service()
    try:
        q = svc.submit(_req("hi", stream=True))
        items = []
        while True:
            items.append(q.get(timeout=5))
            if items[-1]["done"]:
                break
        assert [i["text"] for i in items] == ["ec", "ho:", "hi", ""]
        assert items[-1]["prefill_time"] == 0.25 and items[-1]["decode_tps"] == 50.0
        failed = svc.submit(_req("fail", stream=True)).get(timeout=5)
        assert failed["done"] and failed["error"] == "model_error"
    finally:
        svc.shutdown()


def test_vision_features_are_cached_per_request_id():
    svc = _service()
    try:
        svc.submit(_req("turn 1", rid="conv", images=[b"img-a"])).get(timeout=5)
        svc.submit(_req("turn 2", rid="conv", images=[b"img-a", b"img-b"])).get(timeout=5)
        svc.submit(_req("other", rid="other", images=[b"img-a"])).get(timeout=5)
        feats = svc.contexts.get_or_create("conv").features
        assert feats == [("feat", b"img-a"), ("feat", b"img-b")]  # img-a went through the tower once
        assert [c[3] for c in svc.engine.calls] == [1, 2, 1]
        assert len(svc.contexts) == 2
    finally:
        svc.shutdown()


def test_a_failing_engine_factory_answers_requests_with_the_error():
    def factory():
        raise RuntimeError("CUDA library missing")
    svc = InferenceService(factory, cleanup_every=3600)
    try:
        assert svc.ready.wait(5) and isinstance(svc.failed, RuntimeError)
        r = svc.submit(_req("x")).get(timeout=5)
        assert "CUDA library missing" in r["status"]
    finally:
        svc.shutdown()


# ----------------------------------------------------------------- HTTP layer, as a bare ASGI app
def _asgi(app, method, path, body=None):
    """One request through the ASGI callable; returns (status, headers, body bytes)."""
    payload = b"" if body is None else (body if isinstance(body, bytes) else json.dumps(body).encode())
    scope = {"type": "http", "asgi": {"version": "3.0"}, "http_version": "1.1", "method": method, "path": path,
             "raw_path": path.encode(), "query_string": b"", "root_path": "", "scheme": "http",
             "headers": [(b"content-type", b"application/json"), (b"content-length", str(len(payload)).encode())],
             "client": ("127.0.0.1", 1), "server": ("127.0.0.1", 80)}
    sent = []

    async def run():
        delivered = False

        async def receive():
            nonlocal delivered
            if not delivered:
                delivered = True
                return {"type": "http.request", "body": payload, "more_body": False}
            await asyncio.sleep(3600)

        async def send(message):
            sent.append(message)

        await asyncio.wait_for(app(scope, receive, send), 20)

    asyncio.run(run())
    start = next(m for m in sent if m["type"] == "http.response.start")
    data = b"".join(m.get("body", b"") for m in sent if m["type"] == "http.response.body")
    return start["status"], dict(start["headers"]), data


def test_http_completion_stream_health_and_errors():
    pytest.importorskip("fastapi")
    svc = _service()
    app = serving.create_app(svc, SamplingDefaults(max_new_tokens=16), model_name="m", result_timeout=10)
    try:
        status, _, data = _asgi(app, "GET", "/health")
        assert status == 200 and json.loads(data)["ready"] is True
        # plain completion; the request id is echoed and the timing fields ride along
        status, _, data = _asgi(app, "POST", "/v1/chat/completions",
                                {"messages": [{"role": "user", "content": "hello"}], "request_id": "abc"})
        out = json.loads(data)
        assert status == 200 and out["id"] == "abc" and out["object"] == "chat.completion"
        assert out["choices"][0]["message"] == {"role": "assistant", "content": "echo:hello"}
        assert out["choices"][0]["finish_reason"] == "stop" and out["prefill_time"] == 0.25 and out["decode_tps"] == 100.0
        assert out["usage"]["completion_tokens"] == len("echo:hello") and out["model"] == "m"
        # streaming: server-sent events ending in [DONE]
        status, headers, data = _asgi(app, "POST", "/v1/chat/completions",
                                      {"messages": [{"role": "user", "content": "hi"}], "stream": True})
        assert status == 200 and headers[b"content-type"].startswith(b"text/event-stream")
        events = [e[len("data: "):] for e in data.decode().strip().split("\n\n")]
        assert events[-1] == "[DONE]"
        chunks = [json.loads(e) for e in events[:-1]]
        assert chunks[0]["choices"][0]["delta"] == {"role": "assistant"}
        assert "".join(c["choices"][0]["delta"].get("content", "") for c in chunks) == "echo:hi"
        assert chunks[-1]["choices"][0]["finish_reason"] == "stop" and chunks[-1]["decode_tps"] == 50.0
        # images outside the messages and inside them
        status, _, data = _asgi(app, "POST", "/v1/chat/completions",
                                {"messages": [{"role": "user", "content": [
                                    {"type": "image_url", "image_url": {"url": "data:image/png;base64," + PNG}},
                                    {"type": "text", "text": "describe"}]}], "images": [PNG], "request_id": "im"})
        assert status == 200 and json.loads(data)["choices"][0]["message"]["content"] == "echo:<image>describe"
        assert len(svc.contexts.get_or_create("im").features) == 2
        # client errors
        assert _asgi(app, "POST", "/v1/chat/completions", {"messages": []})[0] == 400
        assert _asgi(app, "POST", "/v1/chat/completions", b"{not json")[0] == 400
        status, _, data = _asgi(app, "POST", "/v1/chat/completions",
                                {"messages": [{"role": "user", "content": "x"}], "images": ["@@@"]})
        assert status == 400 and "failed to decode image" in json.loads(data)["detail"]
        # engine errors become 500 with the engine's code
        status, _, data = _asgi(app, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "fail"}]})
        assert status == 500 and json.loads(data)["detail"] == "model_error"
        strict = serving.create_app(svc, require_images=True, result_timeout=10)
        assert _asgi(strict, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}]})[0] == 400
    finally:
        svc.shutdown()


# ----------------------------------------------------------------- the decoder behind the interface
def test_decoder_engine_generates_through_the_service_on_cpu():
    from cider_b200.decoder import Decoder, DecoderConfig
    tiny = DecoderConfig(hidden=64, layers=2, n_q=4, n_kv=2, head_dim=16, inter=128, vocab=300,
                         mrope_section=(4, 2, 2), tie_embeddings=True)
    vision_calls = []

    def vision(image: bytes):
        vision_calls.append(image)
        g = torch.Generator().manual_seed(len(image))
        return torch.randn(4, 64, generator=g) * 0.02, (1, 2, 2)

    def factory():
        dec = Decoder(tiny, mode="fp16", device="cpu", dtype=torch.float32, max_len=256)
        return serving.DecoderEngine(dec, vision=vision, max_new_tokens=6, use_graph=False, stream_chunk=2)

    svc = InferenceService(factory, cleanup_every=3600)
    try:
        assert svc.ready.wait(30) and svc.failed is None
        msgs = [{"role": "user", "content": "<image>what?"}]
        r1 = svc.submit(InferenceRequest("c", msgs, [b"img"], {"stream": False, "max_new_tokens": 4})).get(timeout=60)
        assert r1["status"] == SUCCESS and len(r1["text"]) == 4 and r1["prefill_time"] > 0 and r1["decode_tps"] > 0
        # the same conversation again: same greedy text, the vision tower is not called again
        r2 = svc.submit(InferenceRequest("c", msgs, [b"img"], {"stream": False, "max_new_tokens": 4})).get(timeout=60)
        assert r2["text"] == r1["text"] and vision_calls == [b"img"]
        # the positions of the prompt follow the text / image / text layout
        embeds, pos3 = svc.engine._inputs(msgs, [b"img"], [torch.zeros(4, 64)], [(1, 2, 2)])
        n_text0 = len("<|user|>")
        assert embeds.shape[1] == pos3.shape[1] and pos3[:, n_text0:n_text0 + 4].tolist() == \
            [[n_text0] * 4, [n_text0, n_text0, n_text0 + 1, n_text0 + 1], [n_text0, n_text0 + 1, n_text0, n_text0 + 1]]
        # streaming cuts the same text into pieces
        q = svc.submit(InferenceRequest("c", msgs, [b"img"], {"stream": True, "max_new_tokens": 4}))
        pieces = []
        while True:
            item = q.get(timeout=60)
            if item["done"]:
                break
            pieces.append(item["text"])
        assert "".join(pieces) == r1["text"] and all(len(p) <= 2 for p in pieces)
        with_too_many = svc.submit(InferenceRequest("d", [{"role": "user", "content": "<image><image>"}], [b"img"],
                                                    {"stream": False})).get(timeout=60)
        assert "more <image> placeholders than images" in with_too_many["status"]
    finally:
        svc.shutdown()
