"""Lazy multi-file safetensors access with nested key prefixes."""
import pytest
import torch

from eridiffusion_b200.io import safetensors as st
from eridiffusion_b200.io.lazy import LazyLoader


def test_lazy_loader_prefixes_and_module_load(tmp_path):
    torch.manual_seed(0)
    lin = torch.nn.Linear(8, 4)
    a = {"blocks.0.attn.weight": torch.randn(4, 8), "blocks.0.attn.bias": torch.randn(4),
         "blocks.1.attn.weight": torch.randn(4, 8).bfloat16()}
    b = {"head.weight": lin.weight.detach().clone(), "head.bias": lin.bias.detach().clone()}
    st.save_file(a, tmp_path / "model-00001.safetensors")
    st.save_file(b, tmp_path / "model-00002.safetensors")
    with LazyLoader(tmp_path) as ld:
        assert sorted(ld.keys()) == sorted(list(a) + list(b)) and ld.has_key("head.bias") and not ld.has_key("nope")
        assert ld.tensor_meta("blocks.1.attn.weight") == ((4, 8), torch.bfloat16) and ld.tensor_meta("x") is None
        assert ld.bytes_read == 0                                   # nothing read so far
        blk = ld.pp("blocks").pp("0")
        assert sorted(blk.keys()) == ["attn.bias", "attn.weight"]
        assert torch.equal(blk.tensor("attn.weight"), a["blocks.0.attn.weight"]) and ld.bytes_read == 4 * 8 * 4
        assert blk.pp("attn").load_tensor("bias", dtype=torch.bfloat16).dtype == torch.bfloat16
        with pytest.raises(ValueError):
            ld.load_tensor("head.weight", shape=(8, 4))
        with pytest.raises(KeyError):
            ld.load_tensor("missing")
        fresh = torch.nn.Linear(8, 4)
        assert ld.pp("head").load_into(fresh) == ([], [])
        assert torch.equal(fresh.weight, lin.weight) and torch.equal(fresh.bias, lin.bias)
        with pytest.raises(KeyError):
            ld.pp("blocks.0.attn").load_into(torch.nn.Linear(8, 4, bias=False))
        d = ld.load_prefix("blocks.1.")
        assert list(d) == ["attn.weight"]
    st.save_file({"head.bias": torch.zeros(4)}, tmp_path / "model-00003.safetensors")
    with pytest.raises(KeyError, match="appears in both"):
        LazyLoader(tmp_path)
