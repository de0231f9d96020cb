"""Inference-time model optimisation: weight quantisation, pruning, memory policy, profiling.

Reference: ``ModelOptimizer`` with ``OptimizationConfig{quantization, pruning, fusion, compilation,
memory_optimization}``, ``OptimizationStats``, ``profile_model`` -> ``ModelProfile{avg_latency_ms,
p99_latency_ms, peak_memory_mb, throughput}`` and ``estimate_model_size``
(crates/inference/src/optimization.rs:11-575).

What each section means here:

* quantisation -- weight-only int8 / int4 / NF4 of the frozen projections through
  ``memory.quantize_model`` (the GEMM operand is expanded by the dequantisation kernel); ``bits``
  selects the format. The reference's calibration-based methods (static, GPTQ, AWQ) need activation
  statistics: calibration batches are accepted and used for a per-layer output-error report, the
  weights are quantised by the same absmax rule.
* pruning -- magnitude / L1 / L2 / random masks, element-wise or structured (whole output rows),
  applied in place to ``Linear`` weights. Gradient- and Taylor-based scores use ``weight * grad``
  when gradients are present and fall back to magnitude.
* fusion -- the framework's layers are already fused (norm + modulate, QK-norm + RoPE, GEMM
  epilogues); the section is reported, there is nothing to rewrite.
* compilation -- no tracing compiler is used on the hot path; a request for one is rejected.
* memory -- attention slicing maps to the chunked attention's key block, CPU offload to the block
  swap manager; both are recorded in the returned plan for the pipeline to apply.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import torch
import torch.nn as nn


@dataclass
class QuantizationConfig:
    method: str = "dynamic"                 # dynamic | static | gptq | awq (see module docstring)
    bits: int = 8
    calibration_samples: int = 0
    symmetric: bool = True
    per_channel: bool = True
    nf4: bool = False                       # 4-bit only: NF4 code book instead of linear int4


@dataclass
class PruningConfig:
    method: str = "magnitude"               # magnitude | l1 | l2 | random | gradient | taylor
    sparsity: float = 0.5
    structured: bool = False
    min_numel: int = 1 << 10


@dataclass
class FusionConfig:
    fuse_conv_bn: bool = True
    fuse_linear_relu: bool = True
    fuse_attention: bool = False
    fuse_layernorm: bool = True


@dataclass
class MemoryConfig:
    gradient_checkpointing: bool = False
    cpu_offload: bool = False
    sequential_cpu_offload: bool = False
    attention_slicing: int | None = None
    vae_slicing: bool = False


@dataclass
class OptimizationConfig:
    quantization: QuantizationConfig | None = None
    pruning: PruningConfig | None = None
    fusion: FusionConfig = field(default_factory=FusionConfig)
    compilation: dict | None = None
    memory_optimization: MemoryConfig = field(default_factory=MemoryConfig)


@dataclass
class OptimizationStats:
    original_bytes: int = 0
    optimized_bytes: int = 0
    quantized_layers: int = 0
    pruned_layers: int = 0
    sparsity: float = 0.0
    calibration_error: dict = field(default_factory=dict)
    memory_plan: dict = field(default_factory=dict)
    notes: list = field(default_factory=list)

    @property
    def compression_ratio(self):
        return self.original_bytes / max(1, self.optimized_bytes)


@dataclass
class ModelProfile:
    avg_latency_ms: float
    p99_latency_ms: float
    peak_memory_mb: float
    throughput: float


def _model_bytes(model) -> int:
    seen, total = set(), 0
    for t in list(model.parameters()) + list(model.buffers()):
        if t.data_ptr() not in seen:
            seen.add(t.data_ptr())
            total += t.numel() * t.element_size()
    for m in model.modules():                      # packed weights of quantised layers
        q = getattr(m, "q", None)
        if q is not None and hasattr(q, "data"):
            total += q.data.numel() * q.data.element_size() + q.scale.numel() * q.scale.element_size()
    return total


class ModelOptimizer:
    def __init__(self, config: OptimizationConfig | None = None):
        self.config = config or OptimizationConfig()
        self.stats = OptimizationStats()
        self.calibration: list = []

    def add_calibration_data(self, data):
        self.calibration.extend(data)

    # ------------------------------------------------------------------ entry point
    def optimize_model(self, model: nn.Module):
        cfg = self.config
        if cfg.compilation:
            raise ValueError("compilation back ends are not supported: kernels are hand-written for sm_100a "
                             "and launched directly")
        st = self.stats = OptimizationStats(original_bytes=_model_bytes(model))
        if cfg.pruning is not None:
            self._prune(model, cfg.pruning)
        if cfg.quantization is not None:
            self._quantize(model, cfg.quantization)
        f = cfg.fusion
        st.notes.append("fusion: norm+modulate, qk-norm+rope, bias/activation/gate/residual epilogues are built in"
                        + ("" if not f.fuse_conv_bn else "; conv+bn: no batch norm in these models"))
        m = cfg.memory_optimization
        st.memory_plan = {"attention_kv_chunk": m.attention_slicing, "block_swap": m.cpu_offload or m.sequential_cpu_offload,
                          "blocks_resident": 1 if m.sequential_cpu_offload else None, "vae_tiling": m.vae_slicing,
                          "activation_checkpointing": m.gradient_checkpointing}
        st.optimized_bytes = _model_bytes(model)
        return model

    # ------------------------------------------------------------------ pruning
    @torch.no_grad()
    def _prune(self, model, pc: PruningConfig):
        from ..models.layers import Linear
        if not 0.0 <= pc.sparsity < 1.0:
            raise ValueError("sparsity must be in [0, 1)")
        zeros = total = 0
        for mod in model.modules():
            if not isinstance(mod, (Linear, nn.Linear)) or mod.weight.numel() < pc.min_numel:
                continue
            w = mod.weight
            score = self._score(w, pc.method)
            if pc.structured:
                row = score.sum(dim=1) if pc.method != "l2" else score.pow(2).sum(dim=1).sqrt()
                k = int(pc.sparsity * row.numel())
                if k:
                    idx = torch.topk(row, k, largest=False).indices
                    w[idx] = 0
                    if getattr(mod, "bias", None) is not None:
                        mod.bias[idx] = 0
            else:
                k = int(pc.sparsity * w.numel())
                if k:
                    th = torch.kthvalue(score.flatten().float(), k).values
                    w.mul_((score > th).to(w.dtype))
            zeros += int((w == 0).sum())
            total += w.numel()
            self.stats.pruned_layers += 1
        self.stats.sparsity = zeros / max(1, total)

    @staticmethod
    def _score(w, method):
        if method in ("magnitude", "l1", "l2", "lottery"):
            return w.abs().float()
        if method == "random":
            return torch.rand(w.shape, device=w.device)
        if method in ("gradient", "taylor"):
            if w.grad is None:
                return w.abs().float()
            return (w * w.grad).abs().float() if method == "taylor" else w.grad.abs().float()
        raise ValueError(f"unknown pruning method {method!r}")

    # ------------------------------------------------------------------ quantisation
    def _quantize(self, model, qc: QuantizationConfig):
        from ..memory import quantize_model
        kind = {8: "int8", 4: "nf4" if qc.nf4 else "int4"}.get(qc.bits)
        if kind is None:
            raise ValueError(f"unsupported weight width {qc.bits} (8 or 4)")
        ref = None
        if self.calibration:
            with torch.no_grad():
                ref = [self._call(model, b) for b in self.calibration[: max(1, qc.calibration_samples or 1)]]
        model.requires_grad_(False)               # inference: every projection is a frozen base weight
        self.stats.quantized_layers = quantize_model(model, kind, min_numel=1 << 10)
        if qc.method != "dynamic":
            self.stats.notes.append(f"quantization method {qc.method!r}: weights use the block-wise absmax rule; "
                                    "calibration data is used for the error report only")
        if ref is not None:
            with torch.no_grad():
                errs = []
                for b, r in zip(self.calibration, ref):
                    o = self._call(model, b)
                    errs.append(float((o.float() - r.float()).norm() / r.float().norm().clamp_min(1e-12)))
            self.stats.calibration_error = {"relative_l2_mean": sum(errs) / len(errs), "relative_l2_max": max(errs)}

    @staticmethod
    def _call(model, batch):
        if isinstance(batch, dict):
            return model(**batch)
        if isinstance(batch, (tuple, list)):
            return model(*batch)
        return model(batch)

    def get_stats(self) -> OptimizationStats:
        return self.stats

    # ------------------------------------------------------------------ profiling
    @staticmethod
    @torch.no_grad()
    def profile_model(model, sample_input, num_runs: int = 20, warmup: int = 3, batch_size: int | None = None):
        """Latency per call over ``num_runs`` (device-timed with CUDA events when the input is on a
        GPU), peak allocator memory and throughput in samples per second."""
        first = sample_input[0] if isinstance(sample_input, (tuple, list)) else (
            next(iter(sample_input.values())) if isinstance(sample_input, dict) else sample_input)
        cuda = first.is_cuda
        bs = batch_size or first.shape[0]
        for _ in range(warmup):
            ModelOptimizer._call(model, sample_input)
        times = []
        if cuda:
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats()
            for _ in range(num_runs):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                ModelOptimizer._call(model, sample_input)
                b.record()
                b.synchronize()
                times.append(a.elapsed_time(b))
            peak = torch.cuda.max_memory_allocated() / 2 ** 20
        else:
            for _ in range(num_runs):
                t0 = time.perf_counter()
                ModelOptimizer._call(model, sample_input)
                times.append((time.perf_counter() - t0) * 1e3)
            peak = 0.0
        times.sort()
        avg = sum(times) / len(times)
        p99 = times[min(len(times) - 1, int(round(0.99 * (len(times) - 1))))]
        return ModelProfile(avg, p99, peak, bs * 1e3 / max(avg, 1e-9))

    @staticmethod
    def estimate_model_size(num_parameters: int, dtype=torch.bfloat16, quantization: QuantizationConfig | None = None):
        bpp = torch.empty((), dtype=dtype).element_size()
        base = num_parameters * bpp
        return base * quantization.bits // (bpp * 8) if quantization else base
