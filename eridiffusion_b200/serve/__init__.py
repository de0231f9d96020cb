"""Inference serving: request queue, dynamic batching, result cache, performance monitor and an
HTTP front end.

Mirrors the reference's inference crate (crates/inference/src/server.rs:165-215 routes
``/v1/txt2img``, ``/v1/img2img``, ``/v1/inpaint``, ``/v1/status/:id``, ``/health``, ``/metrics``;
``BatchInferenceEngine`` with ``DynamicBatchOptimizer`` / ``RequestPrioritizer`` (batch.rs),
``InferenceCache``, ``PerformanceMonitor`` (monitoring.rs)). The reference's accept loop is empty
(server.rs:183-191); here the worker thread really drains the queue. The generator is any callable
``generate(requests: list[GenerationRequest]) -> list[bytes | tensor]`` so the server is
model-agnostic (``sampling.generate_flow`` for MMDiT families).
"""
from __future__ import annotations

import hashlib
import heapq
import itertools
import json
import threading
import time
import uuid
from collections import OrderedDict, deque
from dataclasses import dataclass, field


@dataclass
class GenerationRequest:
    prompt: str = ""
    negative_prompt: str = ""
    width: int = 1024
    height: int = 1024
    steps: int = 20
    guidance_scale: float = 3.5
    seed: int = 0
    mode: str = "txt2img"              # txt2img | img2img | inpaint
    strength: float = 0.8
    priority: int = 0
    init_image: bytes | None = None
    mask: bytes | None = None
    id: str = field(default_factory=lambda: uuid.uuid4().hex)
    submitted: float = field(default_factory=time.time)

    def cache_key(self):
        h = hashlib.sha256()
        h.update(json.dumps([self.prompt, self.negative_prompt, self.width, self.height, self.steps,
                             self.guidance_scale, self.seed, self.mode, self.strength]).encode())
        for b in (self.init_image, self.mask):
            h.update(b or b"")
        return h.hexdigest()

    def batch_key(self):
        return (self.mode, self.width, self.height, self.steps)


class InferenceCache:
    def __init__(self, capacity=256):
        self.capacity, self.data = capacity, OrderedDict()
        self.hits = self.misses = 0

    def get(self, key):
        if key in self.data:
            self.data.move_to_end(key)
            self.hits += 1
            return self.data[key]
        self.misses += 1
        return None

    def put(self, key, value):
        self.data[key] = value
        self.data.move_to_end(key)
        while len(self.data) > self.capacity:
            self.data.popitem(last=False)


class PerformanceMonitor:
    def __init__(self, window=256):
        self.lat = deque(maxlen=window)
        self.batch_sizes = deque(maxlen=window)
        self.total = self.errors = 0
        self.started = time.time()

    def record(self, latency_s, batch):
        self.lat.append(latency_s)
        self.batch_sizes.append(batch)
        self.total += batch

    def snapshot(self):
        lat = sorted(self.lat)
        pick = lambda q: lat[min(len(lat) - 1, int(q * len(lat)))] if lat else 0.0
        return {"requests_total": self.total, "errors_total": self.errors, "latency_p50_s": pick(0.5),
                "latency_p95_s": pick(0.95), "mean_batch": sum(self.batch_sizes) / max(1, len(self.batch_sizes)),
                "uptime_s": time.time() - self.started}

    def prometheus(self):
        s = self.snapshot()
        return "".join(f"eridiffusion_{k} {v}\n" for k, v in s.items())


class DynamicBatcher:
    """Priority queue grouped by ``batch_key``; a batch closes when it is full or when its oldest
    request has waited ``max_wait_s``."""

    def __init__(self, max_batch=4, max_wait_s=0.05):
        self.max_batch, self.max_wait = max_batch, max_wait_s
        self.heap, self.counter = [], itertools.count()
        self.cv = threading.Condition()

    def submit(self, req: GenerationRequest):
        with self.cv:
            heapq.heappush(self.heap, (-req.priority, next(self.counter), req))
            self.cv.notify()

    def next_batch(self, timeout=1.0):
        with self.cv:
            if not self.heap and not self.cv.wait(timeout):
                return []
            if not self.heap:
                return []
            _, _, first = heapq.heappop(self.heap)
            batch = [first]
            deadline = first.submitted + self.max_wait
            while len(batch) < self.max_batch:
                same = [item for item in self.heap if item[2].batch_key() == first.batch_key()]
                if same:
                    item = min(same)
                    self.heap.remove(item)
                    heapq.heapify(self.heap)
                    batch.append(item[2])
                    continue
                left = deadline - time.time()
                if left <= 0 or not self.cv.wait(left):
                    break
            return batch


class InferenceEngine:
    def __init__(self, generate, max_batch=4, max_wait_s=0.05, cache_capacity=256):
        self.generate = generate
        self.batcher = DynamicBatcher(max_batch, max_wait_s)
        self.cache = InferenceCache(cache_capacity)
        self.monitor = PerformanceMonitor()
        self.status = {}
        self.results = {}
        self._stop = threading.Event()
        self.worker = threading.Thread(target=self._loop, daemon=True)

    def start(self):
        self.worker.start()
        return self

    def stop(self):
        self._stop.set()

    def submit(self, req: GenerationRequest):
        cached = self.cache.get(req.cache_key())
        if cached is not None:
            self.status[req.id], self.results[req.id] = "done", cached
            return req.id
        self.status[req.id] = "queued"
        self.batcher.submit(req)
        return req.id

    def _loop(self):
        while not self._stop.is_set():
            batch = self.batcher.next_batch(0.2)
            if not batch:
                continue
            t0 = time.time()
            for r in batch:
                self.status[r.id] = "running"
            try:
                outs = self.generate(batch)
                for r, o in zip(batch, outs):
                    self.results[r.id] = o
                    self.status[r.id] = "done"
                    self.cache.put(r.cache_key(), o)
                self.monitor.record(time.time() - t0, len(batch))
            except Exception as e:           # a failed batch must not kill the worker
                self.monitor.errors += len(batch)
                for r in batch:
                    self.status[r.id] = f"error: {e}"

    def wait(self, rid, timeout=60.0):
        t0 = time.time()
        while time.time() - t0 < timeout:
            st = self.status.get(rid, "unknown")
            if st == "done" or st.startswith("error"):
                return st, self.results.get(rid)
            time.sleep(0.005)
        return "timeout", None


_REQ_MODEL = None


def _request_model():
    """pydantic schema of a generation request (built lazily: pydantic is only needed by the HTTP
    front end)."""
    global _REQ_MODEL
    if _REQ_MODEL is None:
        from pydantic import create_model
        _REQ_MODEL = create_model("Txt2Img", prompt=(str, ...), negative_prompt=(str, ""), width=(int, 1024),
                                  height=(int, 1024), steps=(int, 20), guidance_scale=(float, 3.5),
                                  seed=(int, 0), priority=(int, 0), sync=(bool, False), strength=(float, 0.8),
                                  image=(str | None, None), mask=(str | None, None))
    return _REQ_MODEL


def create_app(engine: InferenceEngine):
    """FastAPI application with the reference's routes."""
    from fastapi import Body, FastAPI, HTTPException
    from fastapi.responses import PlainTextResponse, Response

    app = FastAPI(title="eridiffusion_b200 inference")
    Txt2Img = _request_model()

    def _submit(body, mode):
        try:
            d = Txt2Img(**body).model_dump()
        except Exception as e:
            raise HTTPException(422, str(e))
        sync = d.pop("sync", False)
        # images arrive as base64 PNG text (``image``, ``mask``) and are kept as bytes
        import base64
        try:
            img, msk = (base64.b64decode(v) if v else None for v in (d.pop("image", None), d.pop("mask", None)))
        except Exception as e:
            raise HTTPException(422, f"image / mask must be base64: {e}")
        if mode != "txt2img" and img is None:
            raise HTTPException(422, f"{mode} needs an `image`")
        if mode == "inpaint" and msk is None:
            raise HTTPException(422, "inpaint needs a `mask`")
        rid = engine.submit(GenerationRequest(mode=mode, init_image=img, mask=msk, **d))
        if sync:
            st, out = engine.wait(rid)
            if st != "done":
                raise HTTPException(500, st)
            if isinstance(out, (bytes, bytearray)):
                return Response(content=bytes(out), media_type="image/png")
        return {"id": rid, "status": engine.status.get(rid)}

    @app.post("/v1/txt2img")
    def txt2img(body: dict = Body(...)):
        return _submit(body, "txt2img")

    @app.post("/v1/img2img")
    def img2img(body: dict = Body(...)):
        return _submit(body, "img2img")

    @app.post("/v1/inpaint")
    def inpaint(body: dict = Body(...)):
        return _submit(body, "inpaint")

    @app.get("/v1/status/{rid}")
    def status(rid: str):
        if rid not in engine.status:
            raise HTTPException(404, "unknown request id")
        return {"id": rid, "status": engine.status[rid]}

    @app.get("/health")
    def health():
        return {"status": "ok", "queue": len(engine.batcher.heap)}

    @app.get("/metrics", response_class=PlainTextResponse)
    def metrics():
        return engine.monitor.prometheus()

    return app


def serve(engine: InferenceEngine, host="127.0.0.1", port=8000):
    import uvicorn
    engine.start()
    uvicorn.run(create_app(engine), host=host, port=port)
