"""Serving shell around the decoder: an OpenAI-style chat endpoint in front of ONE worker
thread that owns the engine and takes requests in arrival order.

What it mirrors of the reference (behaviour, not code):

* one inference engine per process, built inside the worker thread and used only there
  (vlm_service/server.py:232-262) - here the thread that owns the CUDA context and the
  captured decode graph;
* a FIFO of requests; streaming and non-streaming results travel back through a
  per-request queue as small dicts (vlm_service/server.py:264-339);
* ``w8a8: auto | on | off`` (vlm_service/core_infer.py:129-157): ``off`` never
  quantises, ``on`` must quantise or fail, ``auto`` quantises when the device
  supports it and otherwise serves in fp16 with a log line;
* a per-request-id cache of vision features with a time-to-live, so that the turns of
  one conversation do not run the vision tower again (vlm_service/server.py:133-180);
* request parameters override the configured sampling defaults
  (vlm_service/server.py:437-466); messages are OpenAI chat messages whose content is
  a string or a list of ``text`` / ``image_url`` parts (vlm_service/server.py:382-434).

The engine is an interface (``complete`` / ``complete_stream``); ``DecoderEngine`` puts
``cider_b200.decoder.Decoder`` behind it.  There is no tokenizer or vision tower in
this repository (no checkpoints travel with it): ``DecoderEngine`` takes them as two
callables and ships byte-level stand-ins for demonstrations and tests.
"""

import base64
import binascii
import json
import logging
import queue
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterator, List, Optional, Sequence, Tuple

log = logging.getLogger("cider_b200.serving")

SUCCESS = "success"
IMAGE_TOKEN = "<image>"


# ------------------------------------------------------------------ w8a8 mode
def resolve_w8a8(mode: str, is_available: Callable[[], bool], convert: Callable[[], Any]) -> Tuple[bool, Any]:
    """The ``w8a8`` switch of the service configuration.

    ``off``: nothing is converted.  ``on``: ``convert()`` runs and every failure
    (unsupported device included) is raised.  ``auto``: converts when
    ``is_available()``; an unsupported device or a failing conversion is logged and
    the service goes on unquantised.  Returns (enabled, what convert() returned)."""
    if mode not in ("auto", "on", "off"):
        raise ValueError(f"w8a8 mode must be 'auto', 'on' or 'off' (got {mode!r})")
    if mode == "off":
        return False, None
    if mode == "auto" and not is_available():
        log.info("[W8A8] device has no INT8 tensor-core path here, serving unquantised")
        return False, None
    try:
        if mode == "on" and not is_available():
            raise RuntimeError("w8a8='on' but the INT8 tensor-core path is not available on this device")
        stats = convert()
        log.info("[W8A8] enabled: %s", stats)
        return True, stats
    except Exception as exc:  # noqa: BLE001 - 'auto' must survive any conversion failure
        if mode == "on":
            raise
        log.warning("[W8A8] initialisation failed, serving unquantised: %s", exc)
        return False, None


# ------------------------------------------------------------------ per-request feature cache
class RequestContext:
    """Vision features of the images a conversation (one request id) has sent so far."""

    def __init__(self, request_id: str, now: float):
        self.request_id = request_id
        self.features: List[Any] = []
        self.stack_features: List[Any] = []
        self.created_at = now
        self.last_accessed = now

    def buffers(self, now: float) -> Tuple[List[Any], List[Any]]:
        self.last_accessed = now
        return self.features, self.stack_features


class RequestContextStore:
    """request id -> RequestContext, entries dropped ``ttl`` seconds after their last use."""

    def __init__(self, ttl: float = 3600.0, clock: Callable[[], float] = time.time):
        self.ttl = float(ttl)
        self._clock = clock
        self._lock = threading.Lock()
        self._contexts: Dict[str, RequestContext] = {}

    def get_or_create(self, request_id: str) -> RequestContext:
        with self._lock:
            ctx = self._contexts.get(request_id)
            if ctx is None:
                ctx = self._contexts[request_id] = RequestContext(request_id, self._clock())
            return ctx

    def cleanup(self) -> int:
        now = self._clock()
        with self._lock:
            dead = [k for k, c in self._contexts.items() if now - c.last_accessed > self.ttl]
            for k in dead:
                del self._contexts[k]
        if dead:
            log.info("dropped %d expired request contexts", len(dead))
        return len(dead)

    def __len__(self) -> int:
        with self._lock:
            return len(self._contexts)

    def now(self) -> float:
        return self._clock()


# ------------------------------------------------------------------ messages and parameters
class BadRequest(ValueError):
    """Client error: becomes HTTP 400."""


def decode_image(data: str, fetch: Optional[Callable[[str], bytes]] = None) -> bytes:
    """An image given as ``data:image/...;base64,xxx``, as bare base64, or as an http(s)
    URL (only with a ``fetch`` function: this module opens no connections itself).
    Returns the encoded image bytes; decoding pixels is the vision tower's business."""
    if not isinstance(data, str):
        raise BadRequest(f"invalid image data type {type(data).__name__}: must be a base64 string or a URL")
    if data.startswith("http://") or data.startswith("https://"):
        if fetch is None:
            raise BadRequest("remote image URLs are not enabled on this server")
        return fetch(data)
    payload = data.split(",", 1)[1] if data.startswith("data:image") and "," in data else data
    try:
        raw = base64.b64decode(payload, validate=True)
    except (binascii.Error, ValueError) as exc:
        raise BadRequest(f"failed to decode image: {exc}") from exc
    if not raw:
        raise BadRequest("failed to decode image: empty payload")
    return raw


def parse_messages(messages: Sequence[Dict[str, Any]], external_images: Optional[List[bytes]] = None,
                   fetch: Optional[Callable[[str], bytes]] = None) -> Tuple[List[Dict[str, str]], List[bytes]]:
    """OpenAI chat messages -> ([{role, content: str}], images).  A content list is
    flattened: text parts are concatenated and every ``image_url`` part becomes the
    placeholder ``<image>`` with its image appended to the list (after the images
    passed outside the messages, which keep their order)."""
    parsed: List[Dict[str, str]] = []
    images: List[bytes] = list(external_images or [])
    for msg in messages:
        role, content = msg.get("role"), msg.get("content")
        if not isinstance(role, str):
            raise BadRequest("every message needs a role")
        if isinstance(content, str):
            parsed.append({"role": role, "content": content})
        elif isinstance(content, list):
            parts: List[str] = []
            for item in content:
                kind = item.get("type") if isinstance(item, dict) else None
                if kind == "text":
                    parts.append(str(item.get("text", "")))
                elif kind == "image_url":
                    url = item.get("image_url", {})
                    url = url.get("url") if isinstance(url, dict) else url
                    images.append(decode_image(url, fetch))
                    parts.append(IMAGE_TOKEN)
            if parts:
                parsed.append({"role": role, "content": "".join(parts)})
        else:
            parsed.append({"role": role, "content": str(content)})
    return parsed, images


@dataclass
class SamplingDefaults:
    temperature: float = 1.0
    top_k: Optional[int] = None
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    max_new_tokens: int = 1024


def merge_params(request: Dict[str, Any], defaults: SamplingDefaults) -> Dict[str, Any]:
    """Request values win over the configured defaults; absent or null fields fall back."""
    def pick(key: str, default):
        v = request.get(key)
        return default if v is None else v
    return {
        "temperature": pick("temperature", defaults.temperature),
        "topp": pick("top_p", defaults.top_p),
        "topk": pick("top_k", defaults.top_k),
        "repetition_penalty": pick("repetition_penalty", defaults.repetition_penalty),
        "max_new_tokens": pick("max_tokens", defaults.max_new_tokens),
        "stream": bool(request.get("stream", False)),
    }


# ------------------------------------------------------------------ the worker
@dataclass
class InferenceRequest:
    request_id: str
    messages: List[Dict[str, str]]
    images: List[bytes]
    params: Dict[str, Any]
    results: "queue.Queue[Dict[str, Any]]" = field(default_factory=queue.Queue)

    @property
    def stream(self) -> bool:
        return bool(self.params.get("stream", False))


class InferenceService:
    """One worker thread, one engine, requests in arrival order.

    ``engine_factory`` runs INSIDE the worker thread (the engine's CUDA context, streams
    and captured graphs belong to the thread that uses them); ``ready`` is set when it
    returned, ``failed`` holds the exception when it raised (requests are then answered
    with that error instead of waiting for ever)."""

    def __init__(self, engine_factory: Callable[[], Any], ttl: float = 3600.0,
                 clock: Callable[[], float] = time.time, cleanup_every: float = 300.0):
        self.contexts = RequestContextStore(ttl, clock)
        self._factory = engine_factory
        self._queue: "queue.Queue[Optional[InferenceRequest]]" = queue.Queue()
        self.engine = None
        self.ready = threading.Event()
        self.failed: Optional[BaseException] = None
        self._stop = threading.Event()
        self._cleanup_every = float(cleanup_every)
        self.served = 0
        self._worker = threading.Thread(target=self._run, name="cider-worker", daemon=True)
        self._worker.start()
        self._janitor = threading.Thread(target=self._clean, name="cider-janitor", daemon=True)
        self._janitor.start()

    # -- client side
    def submit(self, request: InferenceRequest) -> "queue.Queue[Dict[str, Any]]":
        if self._stop.is_set():
            raise RuntimeError("service is shut down")
        self._queue.put(request)
        return request.results

    def pending(self) -> int:
        return self._queue.qsize()

    def shutdown(self, timeout: float = 5.0) -> None:
        self._stop.set()
        self._queue.put(None)
        self._worker.join(timeout)

    # -- worker side
    def _clean(self) -> None:
        while not self._stop.wait(self._cleanup_every):
            self.contexts.cleanup()

    def _run(self) -> None:
        try:
            self.engine = self._factory()
        except BaseException as exc:  # noqa: BLE001 - reported to every request below
            self.failed = exc
            log.error("engine failed to load: %s", exc)
        self.ready.set()
        while True:
            req = self._queue.get()
            if req is None or self._stop.is_set():
                return
            try:
                if self.failed is not None:
                    raise RuntimeError(f"engine failed to load: {self.failed}")
                if req.stream:
                    self._serve_stream(req)
                else:
                    self._serve(req)
            except Exception as exc:  # noqa: BLE001 - one bad request must not end the worker
                log.exception("request %s failed", req.request_id)
                req.results.put({"status": str(exc), "error": str(exc), "done": True})
            finally:
                self.served += 1

    def _buffers(self, req: InferenceRequest):
        return self.contexts.get_or_create(req.request_id).buffers(self.contexts.now())

    def _serve(self, req: InferenceRequest) -> None:
        feats, stack = self._buffers(req)
        code, text, timing = self.engine.complete(req.messages, req.images, feats, stack, **req.params)
        out = {"status": code, "text": text if code == SUCCESS else "",
               "prefill_time": timing.get("prefill_time", 0.0), "decode_tps": timing.get("decode_tps", 0.0)}
        if code != SUCCESS:
            out["error"] = code
        req.results.put(out)

    def _serve_stream(self, req: InferenceRequest) -> None:
        feats, stack = self._buffers(req)
        timing: Dict[str, float] = {}
        for code, text, timing in self.engine.complete_stream(req.messages, req.images, feats, stack, **req.params):
            if code != SUCCESS:
                req.results.put({"status": code, "done": True, "error": code,
                                 "prefill_time": timing.get("prefill_time", 0.0),
                                 "decode_tps": timing.get("decode_tps", 0.0)})
                return
            req.results.put({"text": text, "done": False})
        req.results.put({"text": "", "done": True, "prefill_time": timing.get("prefill_time", 0.0),
                         "decode_tps": timing.get("decode_tps", 0.0)})


# ------------------------------------------------------------------ responses
def completion_response(request_id: str, model: str, result: Dict[str, Any], created: Optional[int] = None) -> Dict[str, Any]:
    text = result.get("text", "")
    return {
        "id": request_id, "object": "chat.completion", "created": int(time.time() if created is None else created),
        "model": model,
        "choices": [{"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": "stop"}],
        "usage": {"prompt_tokens": 0, "completion_tokens": len(text), "total_tokens": len(text)},
        "prefill_time": result.get("prefill_time", 0.0), "decode_tps": result.get("decode_tps", 0.0),
    }


def stream_events(results: "queue.Queue[Dict[str, Any]]", request_id: str, model: str,
                  timeout: Optional[float] = None) -> Iterator[str]:
    """Server-sent events for one streaming request: a role chunk, a content chunk per
    piece of text, a final chunk with finish_reason and the timing, then ``[DONE]``."""
    def chunk(delta: Dict[str, Any], finish: Optional[str] = None, extra: Optional[Dict[str, Any]] = None) -> str:
        body = {"id": request_id, "object": "chat.completion.chunk", "created": int(time.time()), "model": model,
                "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
        if extra:
            body.update(extra)
        return f"data: {json.dumps(body, ensure_ascii=False)}\n\n"

    yield chunk({"role": "assistant"})
    while True:
        item = results.get(timeout=timeout)
        if item.get("error"):
            yield f"data: {json.dumps({'error': {'message': str(item['error'])}})}\n\n"
            break
        if item.get("done"):
            yield chunk({}, "stop", {"prefill_time": item.get("prefill_time", 0.0),
                                     "decode_tps": item.get("decode_tps", 0.0)})
            break
        if item.get("text"):
            yield chunk({"content": item["text"]})
    yield "data: [DONE]\n\n"


# ------------------------------------------------------------------ HTTP layer
def create_app(service: InferenceService, defaults: Optional[SamplingDefaults] = None, model_name: str = "cider-b200",
               fetch: Optional[Callable[[str], bytes]] = None, require_images: bool = False,
               result_timeout: Optional[float] = None):
    """FastAPI application: ``POST /v1/chat/completions`` (OpenAI chat completions,
    ``stream`` supported, plus the fields ``request_id``, ``images``, ``top_k``,
    ``repetition_penalty``), ``GET /health``."""
    import asyncio

    from fastapi import FastAPI, HTTPException, Request
    from fastapi.responses import JSONResponse, StreamingResponse

    defaults = defaults or SamplingDefaults()
    app = FastAPI(title="cider_b200 OpenAI-compatible API")

    @app.get("/health")
    async def health():
        return {"ready": service.ready.is_set() and service.failed is None, "pending": service.pending(),
                "served": service.served, "contexts": len(service.contexts)}

    @app.post("/v1/chat/completions")
    async def chat_completions(http_request: Request):
        try:
            body = await http_request.json()
        except Exception as exc:  # noqa: BLE001
            raise HTTPException(status_code=400, detail=f"invalid JSON body: {exc}")
        if not isinstance(body, dict) or not isinstance(body.get("messages"), list) or not body["messages"]:
            raise HTTPException(status_code=400, detail="'messages' must be a non-empty list")
        if not service.ready.is_set():
            raise HTTPException(status_code=503, detail="service not initialised")
        request_id = body.get("request_id") or str(uuid.uuid4())
        model = body.get("model") or model_name
        try:
            external = [decode_image(d, fetch) for d in (body.get("images") or [])]
            messages, images = parse_messages(body["messages"], external, fetch)
        except BadRequest as exc:
            raise HTTPException(status_code=400, detail=str(exc))
        if require_images and not images:
            raise HTTPException(status_code=400, detail="No images found in messages. This model requires images.")
        params = merge_params(body, defaults)
        results = service.submit(InferenceRequest(request_id, messages, images, params))
        if params["stream"]:
            async def events():
                it = stream_events(results, request_id, model, result_timeout)
                loop = asyncio.get_running_loop()
                while True:
                    ev = await loop.run_in_executor(None, next, it, None)
                    if ev is None:
                        return
                    yield ev
            return StreamingResponse(events(), media_type="text/event-stream")
        result = await asyncio.get_running_loop().run_in_executor(None, lambda: results.get(timeout=result_timeout))
        if result.get("status") != SUCCESS:
            raise HTTPException(status_code=500, detail=str(result.get("error", "unknown error")))
        return JSONResponse(completion_response(request_id, model, result))

    return app


# ------------------------------------------------------------------ the decoder behind the interface
class ByteTokenizer:
    """Stand-in tokenizer: UTF-8 bytes as token ids 0..255, ``<image>`` as id 256 (one
    id per image; the engine expands it to the image's feature rows).  Generated ids
    are folded into bytes (id % 256) and decoded leniently."""
    image_id = 256

    def encode_chat(self, messages: Sequence[Dict[str, str]]) -> List[int]:
        ids: List[int] = []
        for m in messages:
            text = f"<|{m['role']}|>{m['content']}\n"
            pieces = text.split(IMAGE_TOKEN)
            for i, piece in enumerate(pieces):
                ids.extend(piece.encode("utf-8"))
                if i + 1 < len(pieces):
                    ids.append(self.image_id)
        ids.extend(b"<|assistant|>")
        return ids

    def decode(self, ids: Sequence[int]) -> str:
        return bytes(int(i) % 256 for i in ids).decode("utf-8", errors="replace")


class DecoderEngine:
    """``cider_b200.decoder.Decoder`` behind the engine interface of the service.

    ``vision(image_bytes) -> (features [n, hidden], (t, h, w))`` stands for the vision
    tower (n = t*h*w merged patches); its results are kept in the request's feature
    buffer, so a later turn of the same request id with the same images does not call
    it again.  Greedy decoding only (the decoder has no sampler): ``temperature``,
    ``topk``, ``topp`` and ``repetition_penalty`` are accepted and ignored."""

    def __init__(self, decoder, tokenizer=None, vision: Optional[Callable[[bytes], Tuple[Any, Tuple[int, int, int]]]] = None,
                 max_new_tokens: int = 64, use_graph: bool = True, stream_chunk: int = 8):
        self.decoder = decoder
        self.tokenizer = tokenizer or ByteTokenizer()
        self.vision = vision or self._hash_vision
        self.max_new_tokens = int(max_new_tokens)
        self.use_graph = use_graph
        self.stream_chunk = int(stream_chunk)

    def _hash_vision(self, image: bytes):
        """Stand-in vision tower: 2 x 2 feature rows seeded by the image bytes."""
        import hashlib

        import torch
        seed = int.from_bytes(hashlib.sha256(image).digest()[:8], "little") % (2 ** 31)
        g = torch.Generator().manual_seed(seed)
        return torch.randn(4, self.decoder.cfg.hidden, generator=g) * 0.02, (1, 2, 2)

    def _inputs(self, messages, images, feats: List[Any], stack: List[Any]):
        import torch

        from .decoder import mrope_position_ids
        while len(feats) < len(images):  # only the images this conversation has not sent before
            f, grid = self.vision(images[len(feats)])
            feats.append(f)
            stack.append(grid)
        ids = self.tokenizer.encode_chat(messages)
        dec = self.decoder
        rows, segments, run, used = [], [], [], 0
        for tok in ids:
            if tok == getattr(self.tokenizer, "image_id", None):
                if used >= len(images):
                    raise BadRequest("more <image> placeholders than images")
                if run:
                    rows.append(dec.embed[torch.tensor(run, device=dec.embed.device)])
                    segments.append(("text", len(run)))
                    run = []
                rows.append(feats[used].to(device=dec.embed.device, dtype=dec.embed.dtype))
                segments.append(("image", stack[used]))
                used += 1
            else:
                run.append(int(tok) % dec.cfg.vocab)
        if run:
            rows.append(dec.embed[torch.tensor(run, device=dec.embed.device)])
            segments.append(("text", len(run)))
        embeds = torch.cat(rows, dim=0)[None]
        return embeds, mrope_position_ids(segments).to(embeds.device)

    def complete(self, messages, images, feats, stack, **params):
        n = int(params.get("max_new_tokens") or self.max_new_tokens)
        n = max(1, min(n, self.max_new_tokens))
        embeds, pos3 = self._inputs(messages, images, feats, stack)
        toks, stats = self.decoder.generate(embeds, pos3, n, use_graph=self.use_graph)
        timing = {"prefill_time": stats["time_to_first_token_s"], "decode_tps": stats["generation_tps"]}
        return SUCCESS, self.tokenizer.decode(toks[0].tolist()), timing

    def complete_stream(self, messages, images, feats, stack, **params):
        code, text, timing = self.complete(messages, images, feats, stack, **params)
        if code != SUCCESS:
            yield code, "", timing
            return
        for i in range(0, len(text), self.stream_chunk):
            yield SUCCESS, text[i:i + self.stream_chunk], timing


def build_decoder_engine(model: str = "qwen3vl2b", w8a8: str = "auto", group_size: int = 0, max_len: int = 4096,
                         max_new_tokens: int = 64, layers: Optional[int] = None, device: str = "cuda"):
    """Engine factory for ``InferenceService``: a random-weight decoder of the named
    architecture, quantised according to the ``w8a8`` switch."""
    from . import ops
    from .decoder import QWEN3_8B, QWEN3_VL_2B, Decoder
    cfg = QWEN3_VL_2B if model == "qwen3vl2b" else QWEN3_8B

    def make(mode: str):
        return Decoder(cfg, mode=mode, group_size=group_size if mode == "w8a8" else 0, device=device,
                       max_len=max_len, batch=1, layers=layers)

    enabled, dec = resolve_w8a8(w8a8, ops.is_available, lambda: make("w8a8"))
    if not enabled:
        dec = make("fp16")
    return DecoderEngine(dec, max_new_tokens=max_new_tokens)
