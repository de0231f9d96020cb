"""Inference client (against the in-process HTTP app) and the inference-time model optimizer."""
import pytest
import torch
import torch.nn as nn


def _transport(test_client):
    def call(method, url, body, timeout):
        path = url.split("://", 1)[1].split("/", 1)[1]
        r = test_client.request(method, "/" + path, json=body)
        return r.status_code, dict(r.headers), r.content
    return call


def test_client_round_trip():
    from fastapi.testclient import TestClient
    from eridiffusion_b200.serve import InferenceEngine, create_app
    from eridiffusion_b200.serve.client import (ClientConfig, InferenceClient, PooledInferenceClient, ServerError,
                                                TextToImageOptions, decode_image, encode_image)
    img = torch.randint(0, 255, (8, 6, 3), dtype=torch.uint8)
    assert torch.equal(decode_image(encode_image(img)), img)
    f = torch.zeros(3, 4, 4)
    assert decode_image(encode_image(f)).shape == (4, 4, 3) and int(decode_image(encode_image(f))[0, 0, 0]) == 128
    seen = []

    def run(reqs):
        seen.extend(reqs)
        return [encode_png(r) for r in reqs]

    def encode_png(r):
        import base64
        return base64.b64decode(encode_image(torch.full((2, 2, 3), len(r.prompt), dtype=torch.uint8)))

    eng = InferenceEngine(run).start()
    try:
        tc = TestClient(create_app(eng))
    except Exception:
        pytest.skip("test client unavailable")
    cl = InferenceClient(ClientConfig(base_url="http://server"), transport=_transport(tc), sleep=lambda s: None)
    assert cl.health_check()["status"] == "ok"
    png = cl.text_to_image("abc", TextToImageOptions(steps=3, width=64, height=64), sync=True)
    assert decode_image(png)[0, 0].tolist() == [3, 3, 3]
    r = cl.image_to_image("edit", img)
    assert cl.wait(r["id"], poll_s=0.01)["status"] == "done"
    r = cl.inpaint("fill", img, torch.zeros(8, 6, 3, dtype=torch.uint8))
    cl.wait(r["id"], poll_s=0.01)
    by_mode = {q.mode: q for q in seen}
    assert set(by_mode) == {"txt2img", "img2img", "inpaint"}
    assert torch.equal(decode_image(by_mode["img2img"].init_image), img) and by_mode["inpaint"].mask is not None
    assert by_mode["txt2img"].steps == 3 and by_mode["img2img"].strength == 0.75
    with pytest.raises(ServerError) as e:
        cl.check_status("nope")
    assert e.value.status == 404
    with pytest.raises(ServerError):
        cl._call("POST", "/v1/inpaint", {"prompt": "x", "image": encode_image(img)})       # no mask
    assert cl.get_metrics()["eridiffusion_requests_total"] >= 3
    pool = PooledInferenceClient("http://server", 3, transport=_transport(tc))
    outs = pool.batch_text_to_image(["a", "bb", "cccc"], TextToImageOptions(width=64, height=64))
    assert [decode_image(o)[0, 0, 0].item() for o in outs] == [1, 2, 4]
    pool.close()
    eng.stop()


def test_client_retries_connection_errors_and_5xx():
    from eridiffusion_b200.serve.client import ClientConfig, InferenceClient, ServerError
    calls, sleeps = [], []

    def flaky(method, url, body, timeout):
        calls.append(url)
        if len(calls) == 1:
            raise ConnectionRefusedError("down")
        if len(calls) == 2:
            return 503, {}, b"busy"
        return 200, {"Content-Type": "application/json"}, b'{"status": "ok"}'
    cl = InferenceClient(ClientConfig(max_retries=3, retry_delay_s=0.5), transport=flaky, sleep=sleeps.append)
    assert cl.health_check() == {"status": "ok"} and sleeps == [0.5, 1.0]
    always = InferenceClient(ClientConfig(max_retries=2), transport=lambda *a: (500, {}, b"boom"), sleep=lambda s: None)
    with pytest.raises(ServerError):
        always.health_check()


def _mlp():
    from eridiffusion_b200.models.layers import Linear
    torch.manual_seed(0)

    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = Linear(64, 128, dtype=torch.float32)
            self.b = Linear(128, 64, dtype=torch.float32)

        def forward(self, x):
            return self.b(self.a(x, act="gelu"))
    m = M()
    for p in m.parameters():
        nn.init.normal_(p, std=0.1)
    return m


def test_optimizer_quantize_prune_profile():
    from eridiffusion_b200.memory import QuantizedLinear
    from eridiffusion_b200.serve.optimize import (MemoryConfig, ModelOptimizer, OptimizationConfig, PruningConfig,
                                                  QuantizationConfig)
    x = torch.randn(4, 64)
    m = _mlp()
    ref = m(x).detach()
    opt = ModelOptimizer(OptimizationConfig(quantization=QuantizationConfig(bits=8, method="static"),
                                            memory_optimization=MemoryConfig(attention_slicing=1024,
                                                                             sequential_cpu_offload=True)))
    opt.add_calibration_data([x])
    opt.optimize_model(m)
    st = opt.get_stats()
    assert st.quantized_layers == 2 and isinstance(m.a, QuantizedLinear)
    assert 3.0 < st.compression_ratio < 4.1
    assert 0 < st.calibration_error["relative_l2_max"] < 0.02
    assert st.memory_plan["attention_kv_chunk"] == 1024 and st.memory_plan["blocks_resident"] == 1
    assert any("static" in n for n in st.notes)
    assert (m(x) - ref).abs().max() < 0.05
    # 4-bit halves it again
    m4 = _mlp()
    o4 = ModelOptimizer(OptimizationConfig(quantization=QuantizationConfig(bits=4, nf4=True)))
    o4.optimize_model(m4)
    assert o4.get_stats().compression_ratio > 5.0
    # pruning
    mp = _mlp()
    op = ModelOptimizer(OptimizationConfig(pruning=PruningConfig(sparsity=0.5)))
    op.optimize_model(mp)
    assert abs(op.get_stats().sparsity - 0.5) < 0.01 and op.get_stats().pruned_layers == 2
    kept = mp.a.weight[mp.a.weight != 0].abs().min()
    assert kept > 0
    ms = _mlp()
    ModelOptimizer(OptimizationConfig(pruning=PruningConfig(sparsity=0.25, structured=True))).optimize_model(ms)
    zero_rows = (ms.a.weight.abs().sum(1) == 0).sum().item()
    assert zero_rows == 32 and (ms.a.bias == 0).sum().item() >= 32
    with pytest.raises(ValueError):
        ModelOptimizer(OptimizationConfig(compilation={"backend": "tensorrt"})).optimize_model(_mlp())
    with pytest.raises(ValueError):
        ModelOptimizer(OptimizationConfig(quantization=QuantizationConfig(bits=3))).optimize_model(_mlp())
    prof = ModelOptimizer.profile_model(_mlp(), x, num_runs=5, warmup=1)
    assert prof.avg_latency_ms > 0 and prof.p99_latency_ms >= prof.avg_latency_ms * 0.5 and prof.throughput > 0
    assert ModelOptimizer.estimate_model_size(1000, torch.bfloat16) == 2000
    assert ModelOptimizer.estimate_model_size(1000, torch.float32, QuantizationConfig(bits=4)) == 500
