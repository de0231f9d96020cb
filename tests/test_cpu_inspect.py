"""Checkpoint inspection from headers only: layout, block counts, adapter kind / rank, listing."""
import json

import torch

from eridiffusion_b200.cli import inspect as I
from eridiffusion_b200.io import safetensors as st


def test_inspect_model_and_adapter_files(tmp_path, capsys):
    model = {f"double_blocks.{i}.img_attn.qkv.weight": torch.zeros(12, 4, dtype=torch.bfloat16) for i in range(3)}
    model.update({f"single_blocks.{i}.linear1.weight": torch.zeros(8, 4) for i in range(5)})
    f = tmp_path / "flux1-dev-tiny.safetensors"
    st.save_file(model, f, {"format": "pt"})
    s = I.summarise(f)
    assert s["layout"].startswith("flux") and s["blocks"] == {"double_blocks": 3, "single_blocks": 5}
    assert s["model_type_from_path"] == "flux_dev" and s["parameters"] == 3 * 48 + 5 * 32
    assert s["dtypes"] == {"bfloat16": 3, "float32": 5} and s["metadata"] == {"format": "pt"} and "adapter" not in s
    lora = {}
    for i in range(2):
        lora[f"lora.blocks.{i:02d}.attn.q.lora.A"] = torch.zeros(16, 64, dtype=torch.bfloat16)
        lora[f"lora.blocks.{i:02d}.attn.q.lora.B"] = torch.zeros(64, 16, dtype=torch.bfloat16)
    g = tmp_path / "step_000010" / "lora.safetensors"
    g.parent.mkdir()
    st.save_file(lora, g, {"step": 10})
    s2 = I.summarise(g.parent)
    assert s2["adapter"] == {"kind": "lora (eri keys)", "ranks": {16: 2}, "targets": ["q"]} and s2["blocks"] == {"blocks": 2}
    assert I.main([str(f), "--keys", "single_blocks.4", "--limit", "5"]) == 0
    out = capsys.readouterr().out
    assert "single_blocks.4.linear1.weight  float32  [8, 4]" in out and "0.00 M parameters" not in out.split("\n")[1]
    assert I.main([str(g), "--json"]) == 0
    assert json.loads(capsys.readouterr().out.strip())["tensors"] == 4
