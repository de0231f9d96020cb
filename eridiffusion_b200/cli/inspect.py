"""Look inside a safetensors checkpoint without loading it:

    python -m eridiffusion_b200.cli.inspect FILE_OR_DIR [--keys PREFIX] [--limit 40] [--json]

Prints the metadata, dtype histogram, total parameter count and size, the detected model family
(from the path and from the key layout), the number of transformer blocks found, and for adapter
files the adapter kind, ranks and target modules. Counterpart of the reference's ``inspect_*`` /
``verify_*`` helper binaries (src/bin/inspect_*.rs) and of ``infer_num_blocks``
(crates/training/src/flux/weights.rs:44-58); only headers are read.
"""
from __future__ import annotations

import argparse
import json
import re
import sys
from collections import Counter
from pathlib import Path

from ..io.safetensors import SafeFile

_LAYOUTS = (
    ("sdxl (original layout)", r"^model\.diffusion_model\.input_blocks\."),
    ("flux / chroma (double + single blocks)", r"^(model\.diffusion_model\.)?double_blocks\.\d+\."),
    ("sd3 / sd3.5 (joint blocks)", r"^(model\.diffusion_model\.)?joint_blocks\.\d+\."),
    ("diffusers transformer", r"^transformer_blocks\.\d+\."),
    ("text encoder", r"^(text_model|encoder\.block|model\.layers)\."),
    ("vae", r"^(first_stage_model\.|encoder\.down|decoder\.up)"),
)
_ADAPTER = (
    # the reference's per-site names come first: "lora.block03.attn.q.lora.A" also ends in ".lora.A"
    ("lora (reference phase-4 keys: lora.blockNN.attn.q.lora.A)", r"^lora\.block\d+\.(attn|mlp)\.\w+\.lora\.[AB]$"),
    ("lora (reference stable keys: lora.blocks.NN.attn.q.A)", r"^lora\.blocks\.(\d+|mid)\.(attn|mlp)\.\w+\.[AB]$"),
    ("lora (reference SDXL keys: blocks.NN.attn1.to_q.A)", r"^blocks\.\d+\.attn[12]\.to_(q|k|v|out\.0)\.[AB]$"),
    ("lora (eri keys)", r"\.lora\.(A|B)$"), ("lora (PEFT keys)", r"\.lora_(A|B)\.weight$"),
    ("lora (kohya keys)", r"\.lora_(down|up)\.weight$"), ("loha", r"\.hada_w[12]_[ab]$"), ("lokr", r"\.lokr_w[12]"),
    ("dora", r"\.(dora_scale|magnitude)$"), ("ia3", r"\.ia3_"),
)


def summarise(path) -> dict:
    p = Path(path)
    files = sorted(p.glob("*.safetensors")) if p.is_dir() else [p]
    if not files:
        raise FileNotFoundError(f"no safetensors files under {path}")
    entries, meta = {}, {}
    for f in files:
        with SafeFile(f) as sf:
            meta.update(sf.metadata or {})
            for k in sf.keys():
                entries[k] = sf.info(k)
    dtypes = Counter(str(dt).replace("torch.", "") for dt, _ in entries.values())
    numel = {k: _prod(shape) for k, (dt, shape) in entries.items()}
    nbytes = sum(n * _itemsize(entries[k][0]) for k, n in numel.items())
    out = {"files": [str(f) for f in files], "tensors": len(entries), "parameters": sum(numel.values()),
           "bytes": nbytes, "dtypes": dict(dtypes), "metadata": meta}
    keys = list(entries)
    out["layout"] = next((name for name, pat in _LAYOUTS if any(re.search(pat, k) for k in keys)), "unknown")
    try:
        from ..sampling.pipelines import ModelType
        out["model_type_from_path"] = ModelType.from_path(p).value
    except ValueError:
        out["model_type_from_path"] = None
    blocks = {}
    for name in ("double_blocks", "single_blocks", "joint_blocks", "transformer_blocks", "blocks", "layers", "block"):
        sep = "" if name == "block" else r"\."          # the phase-4 LoRA names write "block03"
        idx = {int(m.group(1)) for k in keys if (m := re.search(rf"(?:^|\.){name}{sep}(\d+)\.", k))}
        if idx:
            blocks[name] = max(idx) + 1
    out["blocks"] = blocks
    kind = next((name for name, pat in _ADAPTER if any(re.search(pat, k) for k in keys)), None)
    if kind:
        ranks = Counter()
        targets = set()
        for k, (dt, shape) in entries.items():
            if re.search(r"(lora\.A|lora_A\.weight|lora_down\.weight|\.A)$", k) and len(shape) >= 2:
                ranks[shape[0]] += 1
                targets.add(re.sub(r"\.(lora\.A|lora_A\.weight|lora_down\.weight|A)$", "", k).split(".")[-1])
        out["adapter"] = {"kind": kind, "ranks": dict(ranks), "targets": sorted(targets)}
    out["_entries"] = entries
    return out


def _prod(shape):
    n = 1
    for s in shape:
        n *= s
    return n


def _itemsize(dt):
    import torch
    return torch.empty((), dtype=dt).element_size()


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("path")
    ap.add_argument("--keys", default=None, help="list tensors whose name starts with this prefix")
    ap.add_argument("--limit", type=int, default=40)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    s = summarise(a.path)
    entries = s.pop("_entries")
    if a.json:
        print(json.dumps(s))
        return 0
    print(f"{len(s['files'])} file(s), {s['tensors']} tensors, {s['parameters'] / 1e6:.2f} M parameters, "
          f"{s['bytes'] / 2 ** 20:.1f} MiB; dtypes {s['dtypes']}")
    print(f"layout: {s['layout']}; model type from path: {s['model_type_from_path']}; blocks: {s['blocks'] or '-'}")
    if s.get("adapter"):
        ad = s["adapter"]
        print(f"adapter: {ad['kind']}, ranks {ad['ranks']}, targets {ad['targets']}")
    if s["metadata"]:
        print("metadata:", json.dumps(s["metadata"]))
    if a.keys is not None:
        shown = 0
        for k in sorted(entries):
            if k.startswith(a.keys):
                dt, shape = entries[k]
                print(f"  {k}  {str(dt).replace('torch.', '')}  {list(shape)}")
                shown += 1
                if shown >= a.limit:
                    print(f"  ... (limit {a.limit})")
                    break
    return 0


if __name__ == "__main__":
    sys.exit(main())
