"""Pins of the package surface: layer dependencies, public exports, error taxonomy."""
import ast
import os

import pytest

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "torchllmtuner_b200")

# layer -> layers it may import from (inside the package). Lower layers never import higher ones.
ALLOWED = {
    "errors": set(),
    "config": {"errors"},
    "utils": {"errors", "csrc", "config", "ops", "trainer"},          # utils.validate_runtime drives the public API
    "csrc": {"errors"},
    "accelerator": {"errors", "utils", "ops"},                              # the capability registry probes the extension
    "ops": {"errors", "csrc", "utils", "parallel", "models"},          # ops.gemm asks the comm queue; kernel_bench builds an expert stack
    "models": {"errors", "ops", "utils", "parallel", "config", "accelerator"},   # L4 sits on the L1 collectives (balance-loss sums)
    "memory": {"errors", "ops", "utils"},
    "datasets": {"errors", "utils", "config", "components"},
    "components": {"errors", "ops", "utils", "accelerator", "config", "models", "parallel", "datasets"},
    "parallel": {"errors", "ops", "utils", "accelerator", "config", "models", "memory", "csrc"},
    "trainer": {"errors", "ops", "utils", "accelerator", "config", "models", "memory", "parallel", "components", "datasets"},
    "experiments": {"errors", "ops", "utils", "accelerator", "config", "models", "memory", "parallel", "components", "datasets", "trainer"},
}


def _imports(path, layer):
    tree = ast.parse(open(path).read())
    depth_of_file = os.path.relpath(path, ROOT).count(os.sep)
    for node in ast.walk(tree):
        if isinstance(node, ast.ImportFrom):
            if node.level > 0:
                up = node.level - 1
                parts = os.path.relpath(os.path.dirname(path), ROOT).split(os.sep)
                parts = [p for p in parts if p != "."]
                base = parts[:len(parts) - up] if up <= len(parts) else []
                mod = base + (node.module.split(".") if node.module else [])
                if not mod and node.names:
                    for a in node.names:
                        yield a.name
                elif mod:
                    yield mod[0]
            elif node.module and node.module.startswith("torchllmtuner_b200."):
                yield node.module.split(".")[1]


def test_layer_dependencies():
    bad = []
    for d, _, files in os.walk(ROOT):
        if "__pycache__" in d:
            continue
        rel = os.path.relpath(d, ROOT)
        layer = rel.split(os.sep)[0] if rel != "." else None
        for f in files:
            if not f.endswith(".py"):
                continue
            path = os.path.join(d, f)
            this = layer or os.path.splitext(f)[0]
            if this not in ALLOWED:
                continue
            for target in _imports(path, this):
                target = target.replace(".py", "")
                if target in ALLOWED and target != this and target not in ALLOWED[this]:
                    bad.append(f"{os.path.relpath(path, ROOT)} imports {target}")
    assert not bad, bad
    # the strict bottom of the stack
    assert ALLOWED["config"] == {"errors"} and ALLOWED["errors"] == set()


def test_package_exports_and_lazy_import():
    import torchllmtuner_b200 as pkg
    assert {"LLMTunerConfig", "Trainer"} <= set(dir(pkg)) | set(getattr(pkg, "__all__", []))
    assert pkg.LLMTunerConfig.__name__ == "LLMTunerConfig" and pkg.Trainer.__name__ == "Trainer"
    from torchllmtuner_b200 import ops
    for name in ("linear", "rms_norm", "add_rms_norm", "qk_norm_rope", "swiglu", "attention", "linear_cross_entropy_sum",
                 "cross_entropy_sum", "adamw_step_", "gemm", "AttnMeta", "register_kernel", "get_kernel"):
        assert hasattr(ops, name), name


def test_error_taxonomy():
    from torchllmtuner_b200.errors import (ConfigError, EnvironmentUnsupportedError, KernelStatusError, LLMTunerError,
                                           UnsupportedCombinationError)
    assert issubclass(ConfigError, (LLMTunerError, ValueError))
    assert issubclass(UnsupportedCombinationError, (LLMTunerError, NotImplementedError))
    assert issubclass(EnvironmentUnsupportedError, (LLMTunerError, RuntimeError))
    e = KernelStatusError("gemm", 2, "bounded flag wait expired at site 7401")
    assert isinstance(e, LLMTunerError) and e.code == 2 and "7401" in str(e)
    with pytest.raises(ValueError):
        raise ConfigError("x")
