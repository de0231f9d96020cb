"""The bounds-checked debug build of the kernel library (ERI_B200_DEBUG_BOUNDS=1): the small cases
run clean under it, and an access outside the extent that the host declared is RECORDED AND SKIPPED
(the buffers in these cases are really large enough, only the declared extent is too small, so no
invalid access ever happens — neither with the check nor without it)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]

SCRIPT = r'''
import json, torch
from eridiffusion_b200.ops import _native as N, functional as F
assert N.DEBUG_BOUNDS and str(N._LIB_PATH).endswith("_debug.so")
dev = "cuda"
g = torch.Generator(device=dev).manual_seed(0)
rnd = lambda *s: torch.randn(*s, device=dev, generator=g).bfloat16()
out = {}
# 1. clean runs: GEMM with epilogues, weight gradient, LoRA token reduction, attention, token routing
x, w = rnd(512, 320), rnd(768, 320)
y = F.gemm_native(x, w, bias=rnd(768), act="gelu", pre_out=torch.empty(512, 768, device=dev, dtype=torch.bfloat16))
dw = F.wgrad(rnd(640, 512), rnd(640, 256))
db = F.lora_wgrad(rnd(640, 384), rnd(640, 16))
q, k, v = (rnd(1, 256, 2, 128) for _ in range(3))
o = F.attention(q, k, v)
from eridiffusion_b200.train.act_checkpoint import tread_gather, tread_reinject, tread_select
t = rnd(2, 256, 64)
idx = tread_select(t, k_frac=0.5)
tread_reinject(t, tread_gather(t, idx), idx)
torch.cuda.synchronize()
out["clean"] = N.debug_bounds_report()
out["err"] = F.kernel_error_check()
ref = (x.float() @ w.float().t())
out["gemm_ok"] = bool(torch.isfinite(y.float()).all())
# 2. a declared extent that is too small: the last rows of the output must be left untouched
big = torch.full((512, 768), 7.0, device=dev, dtype=torch.bfloat16)
small = big[:256]                                   # the kernel is told about 256 rows only ...
args = dict(out=big)
import eridiffusion_b200.ops._native as NN
real = NN.extent_bytes
NN.extent_bytes = lambda t: real(t) if t is not big else small.numel() * 2
F.gemm_native(x, w, out=big, force_bn=256)          # ... but computes 512 (two-CTA kernel)
torch.cuda.synchronize()
rep = N.debug_bounds_report()
out["violation"] = rep
out["tail_untouched"] = bool((big[256:] == 7.0).all())
out["head_written"] = bool((big[:256].float() - ref[:256]).abs().max() < 0.5)
big[:256] = 7.0
F.gemm_native(x, w, out=big, force_bn=128)          # the same on the one-CTA kernel
NN.extent_bytes = real
torch.cuda.synchronize()
out["violation1"] = N.debug_bounds_report()
out["tail_untouched1"] = bool((big[256:] == 7.0).all())
out["head_written1"] = bool((big[:256].float() - ref[:256]).abs().max() < 0.5)
# 3. a routing index outside the sequence: skipped and recorded
bad = idx.clone(); bad[0, 0] = 10_000
from eridiffusion_b200.ops import functional as FF
g_out = FF.gather_rows(t, bad)
torch.cuda.synchronize()
out["route"] = N.debug_bounds_report()
print("RESULT " + json.dumps(out))
'''


def test_debug_build_runs_clean_and_records_declared_overruns():
    env = dict(os.environ, ERI_B200_DEBUG_BOUNDS="1", PYTHONPATH=str(ROOT))
    r = subprocess.run([sys.executable, "-c", SCRIPT], env=env, capture_output=True, text=True, timeout=900, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr[-3000:]
    line = next(l for l in r.stdout.splitlines() if l.startswith("RESULT "))
    res = json.loads(line[len("RESULT "):])
    assert res["clean"] == {} and res["err"] == {} and res["gemm_ok"]
    assert list(res["violation"]) == ["gemm2"] and res["violation"]["gemm2"]["code"] == 91 and res["violation"]["gemm2"]["count"] > 0
    assert res["tail_untouched"] and res["head_written"]
    assert list(res["violation1"]) == ["gemm"] and res["violation1"]["gemm"]["code"] == 81 and res["violation1"]["gemm"]["count"] > 0
    assert res["tail_untouched1"] and res["head_written1"]
    assert res["route"]["route"]["code"] == 62 and res["route"]["route"]["value"] == 10_000
