"""Generic checkpoint manager: atomic save, listing, latest / best, convert, merge, extract."""
import json
import os

import pytest
import torch

from eridiffusion_b200.io import safetensors as st
from eridiffusion_b200.train.checkpoint_manager import Checkpoint, CheckpointManager, CheckpointMetadata


def _ck(name, step, loss, scale=1.0):
    return Checkpoint(CheckpointMetadata(name, step=step, loss=loss, model_architecture="flux", network_type="lora"),
                      training_state={"global_step": step}, optimizer_state={"lr": 1e-4}, scheduler_state={"last": step},
                      config={"rank": 4},
                      tensors={"model": {"w": torch.full((2, 3), scale), "idx": torch.tensor([1, 2])},
                               "network": {"lora.A": torch.ones(4, 3, dtype=torch.bfloat16) * scale},
                               "optimizer": {"m": torch.zeros(5)}})


def test_save_load_list_latest_best(tmp_path):
    mgr = CheckpointManager(tmp_path)
    mgr.save_checkpoint(_ck("c20", 20, 0.5, 2.0))
    mgr.save_checkpoint(_ck("c10", 10, 0.7))
    mgr.save_checkpoint(_ck("c30", 30, 0.6, 4.0))
    assert [m.name for m in mgr.list_checkpoints()] == ["c10", "c20", "c30"]
    assert mgr.get_latest_checkpoint() == "c30" and mgr.get_best_checkpoint() == "c20"
    ck = mgr.load_checkpoint("c20")
    assert ck.metadata.step == 20 and ck.training_state == {"global_step": 20} and ck.config == {"rank": 4}
    assert torch.equal(ck.tensors["model"]["w"], torch.full((2, 3), 2.0))
    assert ck.tensors["network"]["lora.A"].dtype == torch.bfloat16 and set(ck.tensors) == {"model", "network", "optimizer"}
    assert set(mgr.load_checkpoint("c20", ("network",)).tensors) == {"network"}
    # a damaged or half-written checkpoint is never listed
    (tmp_path / "c40").mkdir(); (tmp_path / "c40" / "checkpoint.json").write_text("{not json")
    (tmp_path / ".tmp_c50_1").mkdir()
    assert mgr.get_latest_checkpoint() == "c30"
    with pytest.raises(ValueError):
        mgr.save_checkpoint(Checkpoint(CheckpointMetadata("bad"), tensors={"vae": {}}))
    keep = CheckpointManager(tmp_path / "k", keep_last=2)
    for i in range(4):
        keep.save_checkpoint(_ck(f"s{i}", i, 1.0))
    assert [m.name for m in keep.list_checkpoints()] == ["s2", "s3"]


def test_convert_extract_merge(tmp_path):
    mgr = CheckpointManager(tmp_path)
    mgr.save_checkpoint(_ck("a", 1, 0.5, 1.0))
    mgr.save_checkpoint(_ck("b", 2, 0.4, 3.0))
    out = mgr.convert_checkpoint("a", str(tmp_path / "x" / "model_bf16.safetensors"), dtype="bf16")
    t = st.load_file(out)
    assert t["w"].dtype == torch.bfloat16 and t["idx"].dtype == torch.int64
    pt = mgr.convert_checkpoint("a", str(tmp_path / "model.pt"), fmt="pytorch")
    assert torch.equal(torch.load(pt)["w"], torch.ones(2, 3))
    net = mgr.extract_component("b", "network", str(tmp_path / "net.safetensors"))
    assert list(st.load_file(net)) == ["lora.A"] and st.read_metadata(net)["component"] == "network"
    with pytest.raises(ValueError):
        mgr.convert_checkpoint("a", str(tmp_path / "m.onnx"), fmt="onnx")
    with pytest.raises(ValueError):
        mgr.extract_component("a", "vae", str(tmp_path / "v"))
    merged = mgr.merge_checkpoints(["a", "b"], "avg", weights=[1, 3])
    ck = mgr.load_checkpoint("avg")
    assert torch.allclose(ck.tensors["model"]["w"], torch.full((2, 3), 2.5)) and ck.metadata.step == 2
    assert ck.tensors["model"]["idx"].tolist() == [1, 2] and ck.training_state["weights"] == [0.25, 0.75]
    assert os.path.isdir(merged)
    mgr.merge_checkpoints(["a", "b"], "avg_net", component="network")
    assert torch.allclose(mgr.load_checkpoint("avg_net").tensors["network"]["lora.A"].float(), torch.full((4, 3), 2.0))
    with pytest.raises(ValueError):
        mgr.merge_checkpoints(["a", "b"], "bad", weights=[1])
    assert json.load(open(tmp_path / "avg" / "checkpoint.json"))["components"] == ["model"]
