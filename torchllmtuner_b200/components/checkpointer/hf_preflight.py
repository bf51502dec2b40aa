"""Check a Hugging Face model folder against this framework before a run, without reading a single weight
(the reference ships a config/class availability check, examples/hf_model_preflight.py:1-124, and an expert-layout
inspector, examples/inspect_hf_experts.py:1-70; this tool answers the question a run actually asks: will
`--model_name_or_path <folder> --initial_load_path <folder> --initial_load_in_hf true` find every tensor it needs, in the
shape it needs?).

    python -m torchllmtuner_b200.components.checkpointer.hf_preflight <folder> [--json] [--vision]

It reads `config.json`, names the registered model and state format that build it, builds that model on the meta
device, lists the tensor names and shapes the importer will ask for (the state format's `hf_pieces`), and compares them
with the safetensors headers of the folder. Exit code 0 when nothing is missing or mis-shaped.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def expected_tensors(model, stored=None) -> dict[str, tuple[int, ...]]:
    """Hugging Face tensor name -> shape, for every parameter of `model` (built on any device, unsharded). Where a state
    format knows several layouts of a tensor (packed or per-expert files), the one `stored` (names in the folder) holds
    completely is taken, as the importer does; without `stored`, the layout the export writes."""
    from ...models.state import get_state_format
    from .hf import resolve_hf_name
    from .reference_layout import native_shapes
    fmt = get_state_format(getattr(model, "state_format", "native"))
    out: dict[str, tuple[int, ...]] = {}
    for fqn, shape in native_shapes(model).items():
        variants = fmt.hf_piece_variants(fqn, list(shape))
        pick = variants[0]
        if stored is not None:
            pick = next((v for v in variants if all(resolve_hf_name(fmt, pc.name, stored) is not None for pc in v)), pick)
        for piece in pick:
            out[piece.name] = tuple(int(x) for x in piece.shape)
    return out


def stored_tensors(folder: str) -> dict[str, tuple[int, ...]]:
    """Tensor name -> shape from the safetensors headers of `folder` (index file or single file)."""
    from safetensors import safe_open
    from .hf import read_hf_weight_map
    wmap = read_hf_weight_map(folder)
    out: dict[str, tuple[int, ...]] = {}
    for fn in sorted(set(wmap.values())):
        with safe_open(os.path.join(folder, fn), "pt") as f:
            for k in f.keys():
                out[k] = tuple(f.get_slice(k).get_shape())
    return out


_TOWER_FIELDS = ("depth", "hidden_size", "intermediate_size", "num_heads", "in_channels", "patch_size", "spatial_merge_size",
                 "temporal_patch_size", "num_position_embeddings")


def preflight(folder: str, vision: bool = False) -> dict:
    """`vision=True`: a folder whose config.json carries a `vision_config` is checked as the vision-language model (the
    `_vl` entry of its family with the published tower) instead of as its text decoder alone."""
    import torch
    from ...config.model_config import ModelConfig
    from ...models.registry import build_registered_model, registered_models
    from ...models.state import get_state_format, registered_for_hf_model_type
    with open(os.path.join(folder, "config.json")) as f:
        hf = json.load(f)
    key, fmt = registered_for_hf_model_type(hf.get("model_type", ""))
    model_config = ModelConfig(model_name_or_path=folder)
    if vision and key is not None and isinstance(hf.get("vision_config"), dict) and key + "_vl" in registered_models():
        key = key + "_vl"
        arch = fmt.arch_from_hf(hf)
        arch.update(vision_tower="qwen3_5", image_token_id=hf.get("image_token_id", 0),
                    vision=dict({k: hf["vision_config"][k] for k in _TOWER_FIELDS if k in hf["vision_config"]}, patch_order="merge_blocks"))
        for k in ("dtype", "device", "model_config"):
            arch.pop(k, None)
        model_config = ModelConfig(model_name_or_path=key, arch_overrides=arch)
    report = {"folder": folder, "model_type": hf.get("model_type"), "registered_model": key,
              "state_format": getattr(fmt, "name", None), "ok": False}
    if key is None:
        report["error"] = f"model_type {hf.get('model_type')!r} has no registered model"
        return report
    with torch.device("meta"):
        model = build_registered_model(model_config)
    fmt = get_state_format(model.state_format)
    report.update(registered_model=key, state_format=fmt.name)
    report["parameters"] = sum(p.numel() for p in model.parameters())
    try:
        have = stored_tensors(folder)
    except Exception as e:  # noqa: BLE001 - a folder with a config but no weights is a valid thing to ask about
        report.update(error=f"no readable weights: {e}", expected_tensors=len(expected_tensors(model)))
        return report
    want = expected_tensors(model, have)
    from .hf import resolve_hf_name
    found = {k: resolve_hf_name(fmt, k, have) for k in want}          # expected name -> the name it is stored under
    missing = sorted(k for k, v in found.items() if v is None)
    wrong = {k: {"expected": list(want[k]), "stored": list(have[v])} for k, v in sorted(found.items())
             if v is not None and want[k] != have[v]}
    unused = sorted(set(have) - {v for v in found.values() if v is not None})
    report.update(expected_tensors=len(want), stored_tensors=len(have), missing=missing[:50], missing_count=len(missing),
                  shape_mismatches=dict(list(wrong.items())[:50]), shape_mismatch_count=len(wrong),
                  unused=unused[:50], unused_count=len(unused), ok=not missing and not wrong)
    return report


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="hf_preflight", description="check a Hugging Face folder against this framework's importer")
    ap.add_argument("folder")
    ap.add_argument("--json", action="store_true", help="print the whole report as JSON")
    ap.add_argument("--vision", action="store_true", help="check the vision tower's tensors too (folders with a vision_config)")
    a = ap.parse_args(argv)
    rep = preflight(a.folder, vision=a.vision)
    if a.json:
        print(json.dumps(rep, indent=1))
    else:
        print(f"{rep['folder']}: model_type {rep['model_type']} -> model {rep['registered_model']} (state format {rep['state_format']})")
        if "error" in rep:
            print("  " + rep["error"])
        else:
            print(f"  {rep['parameters'] / 1e6:.1f} M parameters, {rep['expected_tensors']} tensors expected, {rep['stored_tensors']} stored")
            for label, key in (("missing", "missing"), ("unused by the importer", "unused")):
                if rep[f"{key}_count"]:
                    print(f"  {label}: {rep[f'{key}_count']}  e.g. {rep[key][:3]}")
            if rep["shape_mismatch_count"]:
                k, v = next(iter(rep["shape_mismatches"].items()))
                print(f"  shape mismatches: {rep['shape_mismatch_count']}  e.g. {k}: expected {v['expected']}, stored {v['stored']}")
        print("  OK" if rep["ok"] else "  NOT OK")
    return 0 if rep["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
