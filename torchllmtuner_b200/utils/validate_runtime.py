"""Offline runtime validator (the role of the reference's `scripts/` validators): `python -m torchllmtuner_b200.utils.validate_runtime`
prints one JSON report of what this machine offers for the framework and exits 0 when the CPU path works (and, on a GPU
box, when the sm_100a extension loads and every visible GPU pair has peer access)."""
from __future__ import annotations

import json
import os
import shutil
import sys


def collect() -> dict:
    import torch
    rep: dict = {"python": sys.version.split()[0], "torch": torch.__version__, "cuda_runtime": torch.version.cuda,
                 "cuda_available": torch.cuda.is_available(), "nvcc": shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"}
    try:
        import torch.distributed as dist
        rep["distributed"] = {"available": dist.is_available(), "nccl": dist.is_nccl_available(), "gloo": dist.is_gloo_available()}
        rep["nccl_version"] = ".".join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else None
    except Exception as e:  # noqa: BLE001
        rep["distributed"] = {"error": str(e)}
    from ..csrc.build import SO_PATH, is_stale
    rep["extension"] = {"path": SO_PATH, "built": os.path.exists(SO_PATH), "stale": is_stale()}
    for mod in ("yaml", "safetensors", "tokenizers", "datasets", "tensorboard"):
        try:
            __import__(mod)
            rep.setdefault("optional", {})[mod] = True
        except Exception:  # noqa: BLE001
            rep.setdefault("optional", {})[mod] = False
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        devs = []
        for i in range(n):
            p = torch.cuda.get_device_properties(i)
            devs.append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                         "memory_gib": round(p.total_memory / 2 ** 30, 1)})
        rep["devices"] = devs
        rep["sm_100"] = all(d["sm"] == "10.0" for d in devs)
        rep["peer_access"] = all(torch.cuda.can_device_access_peer(i, j) for i in range(n) for j in range(n) if i != j)
        try:
            from ..ops.cuda_ext import check_status, load
            ext = load()
            a = torch.randn(256, 128, device="cuda").bfloat16()
            out = torch.empty(256, 256, device="cuda", dtype=torch.bfloat16)
            ext.gemm(a, a, out, False, False, False, 0)
            check_status("validate_runtime")
            err = float((out.float() - a.float() @ a.float().t()).abs().max())
            rep["extension"]["loads"] = True
            rep["extension"]["gemm_max_abs_err"] = err
        except Exception as e:  # noqa: BLE001
            rep["extension"]["loads"] = False
            rep["extension"]["error"] = str(e)[:300]
        try:
            import torch.distributed._symmetric_memory  # noqa: F401
            rep["symmetric_memory"] = True
        except Exception:  # noqa: BLE001
            rep["symmetric_memory"] = False
    # the CPU path: one tiny training step through the public API
    try:
        os.environ.setdefault("LLMTUNER_DEVICE", "cpu") if not torch.cuda.is_available() else None
        from .. import LLMTunerConfig, Trainer
        cfg = LLMTunerConfig()
        cfg.apply_flat(dict(model_name_or_path="qwen3", vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                            num_attention_heads=2, num_key_value_heads=1, global_batch_size=2, max_seq_len=16, steps=1,
                            dump_folder="/tmp/llmt_validate"))
        tr = Trainer(cfg)
        try:
            rep["train_step_loss"] = tr.train_step().loss
        finally:
            tr.close()
    except Exception as e:  # noqa: BLE001
        rep["train_step_error"] = str(e)[:300]
    return rep


def main() -> int:
    rep = collect()
    print(json.dumps(rep, indent=1))
    ok = "train_step_loss" in rep
    if rep.get("cuda_available"):
        ok = ok and rep["extension"].get("loads", False) and (rep.get("peer_access", True) or len(rep.get("devices", [])) < 2)
    return 0 if ok else 1


if __name__ == "__main__":
    raise SystemExit(main())
