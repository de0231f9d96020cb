"""HTTP client of the inference server.

Reference: ``InferenceClient{text_to_image, image_to_image, inpaint, check_status, health_check,
get_metrics}``, option structs, ``AsyncInferenceClient::batch_text_to_image`` over a pool of
connections, and the base64 image helpers (crates/inference/src/client.rs:14-420).

The transport is a callable ``(method, url, json_body, timeout) -> (status, headers, bytes)``; the
default uses ``urllib`` from the standard library, tests pass an in-process one. Images travel as
base64-encoded PNG in the request body (``image``, ``mask``) and come back either as PNG bytes
(``sync`` requests) or through the request id.
"""
from __future__ import annotations

import base64
import io
import json
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import asdict, dataclass

import torch


@dataclass
class ClientConfig:
    base_url: str = "http://127.0.0.1:8000"
    timeout_s: float = 300.0
    max_retries: int = 3
    retry_delay_s: float = 0.5


@dataclass
class TextToImageOptions:
    negative_prompt: str = ""
    width: int = 1024
    height: int = 1024
    steps: int = 20
    guidance_scale: float = 3.5
    seed: int = 0
    priority: int = 0


@dataclass
class ImageToImageOptions(TextToImageOptions):
    strength: float = 0.75


@dataclass
class InpaintOptions(ImageToImageOptions):
    pass


class ServerError(RuntimeError):
    def __init__(self, status, body):
        super().__init__(f"server answered {status}: {body[:200]!r}")
        self.status, self.body = status, body


def _urllib_transport(method, url, body, timeout):
    import urllib.error
    import urllib.request
    data = None if body is None else json.dumps(body).encode()
    req = urllib.request.Request(url, data=data, method=method,
                                 headers={"Content-Type": "application/json"} if data else {})
    try:
        with urllib.request.urlopen(req, timeout=timeout) as r:
            return r.status, dict(r.headers), r.read()
    except urllib.error.HTTPError as e:
        return e.code, dict(e.headers), e.read()


def encode_image(img: torch.Tensor) -> str:
    """uint8 ``[H, W, 3]`` (or float ``[3, H, W]`` in [-1, 1]) -> base64 PNG."""
    from PIL import Image
    if img.dtype != torch.uint8:
        img = ((img.float() + 1) * 0.5).clamp(0, 1).mul(255).round().to(torch.uint8).permute(1, 2, 0)
    buf = io.BytesIO()
    Image.fromarray(img.cpu().numpy()).save(buf, format="PNG")
    return base64.b64encode(buf.getvalue()).decode()


def decode_image(data) -> torch.Tensor:
    """PNG bytes or base64 text -> uint8 ``[H, W, C]``."""
    import numpy as np
    from PIL import Image
    raw = base64.b64decode(data) if isinstance(data, str) else bytes(data)
    return torch.from_numpy(np.array(Image.open(io.BytesIO(raw))))


class InferenceClient:
    def __init__(self, config: ClientConfig | None = None, transport=None, sleep=time.sleep):
        self.config = config or ClientConfig()
        self.transport = transport or _urllib_transport
        self.sleep = sleep

    def _call(self, method, path, body=None):
        c = self.config
        url = c.base_url.rstrip("/") + path
        last = None
        for attempt in range(max(1, c.max_retries)):
            try:
                status, headers, content = self.transport(method, url, body, c.timeout_s)
            except OSError as e:                     # connection refused / reset / timed out
                last = e
                self.sleep(c.retry_delay_s * 2 ** attempt)
                continue
            if status >= 500 and attempt + 1 < c.max_retries:
                last = ServerError(status, content)
                self.sleep(c.retry_delay_s * 2 ** attempt)
                continue
            if status >= 400:
                raise ServerError(status, content)
            ctype = {k.lower(): v for k, v in headers.items()}.get("content-type", "")
            if ctype.startswith("image/"):
                return content
            if ctype.startswith("text/plain"):
                return content.decode()
            return json.loads(content) if content else None
        raise last if last is not None else RuntimeError("request failed")

    # -- generation
    def text_to_image(self, prompt: str, options: TextToImageOptions | None = None, sync: bool = False):
        """Returns PNG bytes when ``sync`` (the server answers with the image), else
        ``{"id", "status"}``."""
        return self._call("POST", "/v1/txt2img", {"prompt": prompt, **asdict(options or TextToImageOptions()),
                                                  "sync": sync})

    def image_to_image(self, prompt: str, image: torch.Tensor, options: ImageToImageOptions | None = None,
                       sync: bool = False):
        return self._call("POST", "/v1/img2img", {"prompt": prompt, "image": encode_image(image),
                                                  **asdict(options or ImageToImageOptions()), "sync": sync})

    def inpaint(self, prompt: str, image: torch.Tensor, mask: torch.Tensor, options: InpaintOptions | None = None,
                sync: bool = False):
        return self._call("POST", "/v1/inpaint", {"prompt": prompt, "image": encode_image(image),
                                                  "mask": encode_image(mask), **asdict(options or InpaintOptions()),
                                                  "sync": sync})

    # -- status
    def check_status(self, request_id: str) -> dict:
        return self._call("GET", f"/v1/status/{request_id}")

    def wait(self, request_id: str, poll_s: float = 0.25, timeout_s: float | None = None) -> dict:
        deadline = time.time() + (timeout_s or self.config.timeout_s)
        while True:
            st = self.check_status(request_id)
            if st["status"] not in ("queued", "running"):
                return st
            if time.time() > deadline:
                raise TimeoutError(f"request {request_id} still {st['status']}")
            self.sleep(poll_s)

    def health_check(self) -> dict:
        return self._call("GET", "/health")

    def get_metrics(self) -> dict:
        """The ``/metrics`` text (Prometheus exposition format) parsed into ``{name: value}``."""
        out = {}
        for line in self._call("GET", "/metrics").splitlines():
            if line and not line.startswith("#"):
                k, _, v = line.rpartition(" ")
                try:
                    out[k] = float(v)
                except ValueError:
                    pass
        return out

    @staticmethod
    def save_response(png_bytes: bytes, path: str):
        with open(path, "wb") as f:
            f.write(png_bytes)
        return path


class PooledInferenceClient:
    """Several requests in flight at once (the reference's ``AsyncInferenceClient`` with
    ``num_connections``); results keep the order of the prompts."""

    def __init__(self, base_url: str, num_connections: int = 4, transport=None):
        self.client = InferenceClient(ClientConfig(base_url=base_url), transport)
        self.pool = ThreadPoolExecutor(max_workers=max(1, num_connections))

    def batch_text_to_image(self, prompts, options: TextToImageOptions | None = None, sync: bool = True):
        futs = [self.pool.submit(self.client.text_to_image, p, options, sync) for p in prompts]
        return [f.result() for f in futs]

    def close(self):
        self.pool.shutdown(wait=True)
