"""Core utilities: typed errors, device parsing, plug-in registry, validation, strict counters."""
import pytest
import torch

from eridiffusion_b200 import utils as U


def test_error_classification_and_comm_timeout_decoding():
    assert isinstance(U.classify_cuda_error(RuntimeError("CUDA out of memory. Tried to allocate")), U.OutOfMemoryError)
    assert isinstance(U.classify_cuda_error(RuntimeError("cuDNN error: CUDNN_STATUS_BAD_PARAM")), U.DeviceError)
    assert type(U.classify_cuda_error(ValueError("something else"))) is U.EriError
    e = U.CommTimeoutError(((1 + 1) << 8) | 3, rank=0)
    assert (e.channel, e.peer) == (1, 3)


def test_device_parse_and_manager_on_cpu():
    assert str(U.Device.parse("cuda:2")) == "cuda:2" and U.Device.parse("cpu").kind == "cpu"
    assert U.Device.parse("3") == U.Device("cuda", 3)
    with pytest.raises(U.DeviceError):
        U.Device.parse("tpu")
    m = U.DeviceManager()
    if not torch.cuda.is_available():
        assert m.device.kind == "cpu" and m.memory()["allocated_mb"] == 0.0
        with pytest.raises(U.DeviceError):
            m.set("cuda:0")
    assert U.now_millis() > 0 and U.memory_mb() >= 0.0


def test_plugin_registry_register_get_and_conflicts():
    reg = U.PluginRegistry()
    reg.register("optimizers", "mine", dict)

    @reg.register("samplers", "s1")
    def make():
        return 7

    assert reg.create("samplers", "s1") == 7 and reg.names("optimizers") == ["mine"]
    with pytest.raises(U.ConfigurationError):
        reg.register("optimizers", "mine", list)
    reg.register("optimizers", "mine", list, override=True)
    with pytest.raises(U.ConfigurationError, match="known: mine"):
        reg.get("optimizers", "absent")
    reg.load("eridiffusion_b200.utils.stability")        # importing a module is a valid plug-in


def test_validation_helpers():
    t = torch.zeros(2, 4, 8, 8)
    U.validate_shape(t, (2, None, (8, 16), 8))
    with pytest.raises(U.ShapeError):
        U.validate_shape(t, (2, 4, 9, 8))
    with pytest.raises(U.ShapeError):
        U.validate_dtype(t, torch.bfloat16)
    with pytest.raises(U.ConfigurationError):
        U.validate_range(1.5, 0.0, 1.0, "p")
    U.validate_train_inputs(t, torch.zeros(2, 7, 16), torch.zeros(2))
    bad = t.clone()
    bad[0, 0, 0, 0] = float("nan")
    with pytest.raises(U.ShapeError, match="1 NaN"):
        U.validate_train_inputs(bad, torch.zeros(2, 7, 16))
    with pytest.raises(U.ConfigurationError):
        U.validate_train_inputs(torch.zeros(2, 4, 7, 8), torch.zeros(2, 7, 16))


def test_strict_scope_counts_clones_casts_and_layout_fixes():
    x = torch.randn(64, 128).bfloat16()
    with U.strict_scope() as c:
        y = x * 2                                   # plain math: nothing counted
        _ = y + 1
    assert c.snapshot() == {"clone_allocs": 0, "f32_graph_casts": 0, "layout_fixes": 0}
    with U.strict_scope() as c:
        _ = x.clone()
        _ = x.float()
        _ = x.t().contiguous()
        _ = torch.ones(4).bfloat16().float()        # tiny tensors are not activations
    assert c.snapshot() == {"clone_allocs": 1, "f32_graph_casts": 1, "layout_fixes": 1}
    with pytest.raises(RuntimeError):
        with U.strict_scope(panic=True):
            x.float()


def test_stability_helpers():
    m = torch.tensor([[True, False]])
    a = U.sanitize_attn_mask(m, torch.float32)
    assert a.tolist() == [[0.0, -1e4]]
    assert U.sanitize_attn_mask(torch.tensor([-1e9, 0.5])).float().tolist() == [-9984.0, 0.0]
    p, t = torch.ones(4).bfloat16(), torch.zeros(4).bfloat16()
    assert U.compute_loss_fp32(p, t).dtype == torch.float32 and float(U.compute_loss_fp32(p, t)) == 1.0
