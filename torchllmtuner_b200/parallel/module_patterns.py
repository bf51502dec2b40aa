"""Module-path patterns shared by the tensor-parallel overrides and the FSDP unit selection
(reference: llmtuner/parallel/module_patterns.py:13-66).

Grammar, matched against the whole dotted module name:
    *          any run of characters (dots included)
    ?          any one character
    {*}        one numeric path segment (digits only)
    {a-b}      one number of the inclusive range a..b, so `model.layers.{0-3}.mlp` names the MLPs of the first four blocks
Any other brace is an error. `resolve_module_patterns` refuses a pattern that selects nothing: a typo must not silently
leave a module out of a plan.
"""
from __future__ import annotations

import re
from functools import lru_cache


@lru_cache(maxsize=512)
def compile_module_pattern(pattern: str) -> re.Pattern:
    out: list[str] = []
    i, n = 0, len(pattern)
    while i < n:
        ch = pattern[i]
        if ch == "{":
            close = pattern.find("}", i)
            if close < 0:
                raise ValueError(f"module pattern {pattern!r}: '{{' without '}}'")
            body = pattern[i + 1:close]
            if body == "*":
                out.append("[0-9]+")
            else:
                lo, sep, hi = body.partition("-")
                if not sep or not lo.isdigit() or not hi.isdigit():
                    raise ValueError(f"module pattern {pattern!r}: '{{{body}}}' is neither '{{*}}' nor a numeric range '{{a-b}}'")
                a, b = int(lo), int(hi)
                if a > b:
                    raise ValueError(f"module pattern {pattern!r}: empty range {{{a}-{b}}}")
                out.append("(?:" + "|".join(str(v) for v in range(a, b + 1)) + ")")
            i = close + 1
            continue
        if ch == "}":
            raise ValueError(f"module pattern {pattern!r}: '}}' without '{{'")
        out.append(".*" if ch == "*" else "." if ch == "?" else re.escape(ch))
        i += 1
    return re.compile("".join(out))


def module_name_matches(name: str, pattern: str) -> bool:
    return compile_module_pattern(pattern).fullmatch(name) is not None


def resolve_module_patterns(names, patterns, plan_name: str = "plan") -> set[str]:
    """Names selected by any of `patterns`; a pattern that selects nothing raises."""
    names = list(names)
    chosen: set[str] = set()
    for pat in patterns:
        rx = compile_module_pattern(pat)
        hit = {n for n in names if rx.fullmatch(n)}
        if not hit:
            raise ValueError(f"{plan_name}: pattern {pat!r} matches no module")
        chosen |= hit
    return chosen
