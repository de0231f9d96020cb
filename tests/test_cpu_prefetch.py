"""Native read-ahead threads: ranges arrive intact and in any wait order, back-pressure holds,
errors come back through wait, tensor payloads of a safetensors file decode from the buffer."""
import threading
import time

import pytest
import torch

from eridiffusion_b200.io import native_host as NH
from eridiffusion_b200.io import safetensors as st

pytestmark = pytest.mark.skipif(NH.lib() is None or not hasattr(NH.lib(), "eri_prefetch_create"),
                                reason="native host library not built")


def test_ranges_and_errors(tmp_path):
    data = bytes(range(256)) * 4096                                  # 1 MiB
    f = tmp_path / "blob.bin"
    f.write_bytes(data)
    with NH.Prefetcher(threads=3, max_inflight=8) as pf:
        tickets = [(pf.submit(f, off, n), off, n) for off, n in ((0, 1000), (4096, 65536), (len(data) - 10, 10), (5, 0))]
        for t, off, n in reversed(tickets):                          # wait in another order than submitted
            got = pf.wait(t)
            assert bytes(got.numpy().tobytes()) == data[off:off + n]
            pf.release(t)
        assert pf.bytes_read() == 1000 + 65536 + 10
        bad = pf.submit(tmp_path / "missing.bin", 0, 16)
        with pytest.raises(OSError, match="cannot open"):
            pf.wait(bad)
        pf.release(bad)
        short = pf.submit(f, len(data) - 4, 64)
        with pytest.raises(OSError, match="short read"):
            pf.wait(short)
        pf.release(short)
        with pytest.raises(ValueError):
            pf.submit(f, -1, 4)


def test_back_pressure_and_safetensors_payload(tmp_path):
    w = torch.randn(64, 33).bfloat16()
    st.save_file({"a": torch.arange(10, dtype=torch.float32), "w": w}, tmp_path / "m.safetensors")
    with NH.Prefetcher(threads=2, max_inflight=2) as pf, st.SafeFile(tmp_path / "m.safetensors") as sf:
        t1, t2 = pf.submit_tensor(sf, "w"), pf.submit_tensor(sf, "a")
        blocked = []

        def third():
            blocked.append(pf.submit_tensor(sf, "a"))                # waits until a ticket is released

        th = threading.Thread(target=third)
        th.start()
        time.sleep(0.3)
        assert not blocked
        got = pf.wait(t1).view(torch.bfloat16).view(64, 33)
        assert torch.equal(got, w)
        pf.release(t1)
        th.join(timeout=10)
        assert len(blocked) == 1
        assert torch.equal(pf.wait(t2).view(torch.float32), torch.arange(10, dtype=torch.float32))
        pf.release(t2)
        pf.release(blocked[0])


def test_cached_tensor_batch_reads_match_plain_reads(tmp_path):
    from eridiffusion_b200.data import load_cached_tensors, save_cached_tensor
    paths = []
    for i, key in enumerate(["latent", "text_embed", "data", "text_hidden"]):
        p = tmp_path / f"t{i}.safetensors"
        t = torch.randn(1, 5 + i, 8) if i % 2 else torch.randn(4, 6, 6).bfloat16()
        save_cached_tensor(p, t, key)
        paths.append(p)
    plain = load_cached_tensors(paths)
    with NH.Prefetcher(threads=2, max_inflight=3) as pf:
        fast = load_cached_tensors(paths, prefetcher=pf)         # 4 files through 3 slots: windowed
    assert all(torch.equal(a, b) and a.dtype == torch.bfloat16 for a, b in zip(plain, fast))
    assert plain[1].shape == (6, 8)                               # leading singleton squeezed
