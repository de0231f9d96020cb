"""Numerical accuracy reports for comparing two implementations of the same op or model.

Reference: ``AccuracyReport{max/mean absolute and relative error, num_elements, tolerance, passed}``
with ``from_vectors`` and ``format_report``, ``AccuracyTestSuite{add_report, add_comparison,
all_passed, num_passed, num_failed, generate_summary, save_to_file}``, ``compare_shapes`` and
``DifferenceStats{num_zeros, num_small (<1e-6), num_medium, num_large (>1e-3), percentile_95,
percentile_99}`` (src/inference/numerical_accuracy.rs:12-309).

All statistics are reduced on the device the tensors live on (one pass, fp32) and only scalars come
back to the host; the reference copies both tensors to host vectors first.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass

import torch


def compare_shapes(name, shape1, shape2):
    if tuple(shape1) != tuple(shape2):
        raise ValueError(f"{name}: shape mismatch {tuple(shape1)} vs {tuple(shape2)}")


@dataclass
class DifferenceStats:
    num_zeros: int
    num_small: int
    num_medium: int
    num_large: int
    percentile_95: float
    percentile_99: float

    @classmethod
    def from_differences(cls, diffs: torch.Tensor):
        d = diffs.detach().float().abs().flatten()
        if d.numel() == 0:
            return cls(0, 0, 0, 0, 0.0, 0.0)
        zeros = int((d == 0).sum())
        small = int(((d > 0) & (d < 1e-6)).sum())
        large = int((d > 1e-3).sum())
        # quantile() is limited to 16M elements: sub-sample evenly beyond that
        q = d if d.numel() <= (1 << 24) else d[:: d.numel() // (1 << 24) + 1]
        p95, p99 = (float(v) for v in torch.quantile(q, torch.tensor([0.95, 0.99], device=q.device)))
        return cls(zeros, small, d.numel() - zeros - small - large, large, p95, p99)

    def format_report(self, total: int | None = None) -> str:
        total = total or (self.num_zeros + self.num_small + self.num_medium + self.num_large) or 1
        pct = lambda n: f"{n} ({100.0 * n / total:.2f}%)"
        return (f"  exact: {pct(self.num_zeros)}\n  <1e-6: {pct(self.num_small)}\n  1e-6..1e-3: {pct(self.num_medium)}\n"
                f"  >1e-3: {pct(self.num_large)}\n  p95 {self.percentile_95:.3e}  p99 {self.percentile_99:.3e}")


@dataclass
class AccuracyReport:
    name: str
    max_absolute_error: float
    mean_absolute_error: float
    max_relative_error: float
    mean_relative_error: float
    num_elements: int
    tolerance: float
    passed: bool
    num_nonfinite: int = 0

    @classmethod
    def from_tensors(cls, name, actual: torch.Tensor, expected: torch.Tensor, tolerance: float = 1e-3,
                     relative_floor: float = 1e-8):
        """``passed``: no non-finite mismatch and max |a - e| <= tolerance * max(1, max |e|)."""
        compare_shapes(name, actual.shape, expected.shape)
        a, e = actual.detach().float(), expected.detach().float().to(actual.device)
        bad = int((~torch.isfinite(a) ^ ~torch.isfinite(e)).sum())
        fin = torch.isfinite(a) & torch.isfinite(e)
        d = (a - e).abs()[fin]
        if d.numel() == 0:
            return cls(name, 0.0, 0.0, 0.0, 0.0, a.numel(), tolerance, bad == 0, bad)
        rel = d / e[fin].abs().clamp_min(relative_floor)
        scale = max(1.0, float(e[fin].abs().max()))
        mx = float(d.max())
        return cls(name, mx, float(d.mean()), float(rel.max()), float(rel.mean()), a.numel(), tolerance,
                   bad == 0 and mx <= tolerance * scale, bad)

    from_vectors = from_tensors

    def format_report(self) -> str:
        return (f"[{'PASS' if self.passed else 'FAIL'}] {self.name}: max abs {self.max_absolute_error:.3e}, "
                f"mean abs {self.mean_absolute_error:.3e}, max rel {self.max_relative_error:.3e}, "
                f"mean rel {self.mean_relative_error:.3e}, n={self.num_elements}, tol {self.tolerance:g}"
                + (f", {self.num_nonfinite} non-finite mismatches" if self.num_nonfinite else ""))


class AccuracyTestSuite:
    def __init__(self):
        self.reports: list[AccuracyReport] = []

    def add_report(self, report: AccuracyReport):
        self.reports.append(report)
        return report

    def add_comparison(self, name, actual, expected, tolerance=1e-3):
        return self.add_report(AccuracyReport.from_tensors(name, actual, expected, tolerance))

    def all_passed(self) -> bool:
        return all(r.passed for r in self.reports)

    def num_passed(self) -> int:
        return sum(r.passed for r in self.reports)

    def num_failed(self) -> int:
        return len(self.reports) - self.num_passed()

    def generate_summary(self) -> str:
        lines = [f"numerical accuracy: {self.num_passed()}/{len(self.reports)} passed"]
        lines += [r.format_report() for r in self.reports]
        return "\n".join(lines)

    def save_to_file(self, path):
        with open(path, "w") as f:
            if str(path).endswith(".json"):
                json.dump({"passed": self.all_passed(), "reports": [asdict(r) for r in self.reports]}, f, indent=1)
            else:
                f.write(self.generate_summary() + "\n")
        return path
