"""Extracts, from the reference project's Python sources, the shape of every call its runtime makes
into its native module ``_C`` -- entry-point name, number of positional arguments, keyword names,
whether ``*args`` / ``**kwargs`` are splatted, and which arguments are wrapped as DLPack capsules --
and writes them to ``reference_native_calls.json`` next to this script.

    python tests/golden/make_native_calls.py /path/to/reference

The fixture pins the calling convention a drop-in native module has to accept
(tests/test_native_signature_cpu.py binds each recorded call against this library's native object).
Only call shapes are recorded, no source text.
"""
from __future__ import annotations

import ast
import json
import sys
from pathlib import Path


def _is_native_call(node: ast.Call) -> str | None:
    f = node.func
    # _backend._C.<name>(...)
    if (isinstance(f, ast.Attribute) and isinstance(f.value, ast.Attribute)
            and f.value.attr == "_C"):
        return f.attr
    return None


def _wrapped(arg: ast.expr) -> bool:
    """True when the argument expression is (or conditionally is) wrap_for_dlpack(...)."""
    for sub in ast.walk(arg):
        if isinstance(sub, ast.Call):
            fn = sub.func
            name = fn.attr if isinstance(fn, ast.Attribute) else getattr(fn, "id", "")
            if name == "wrap_for_dlpack":
                return True
    return False


def extract(root: Path):
    calls = []
    for path in sorted((root / "src" / "risa_attention").glob("*.py")):
        tree = ast.parse(path.read_text())
        for node in ast.walk(tree):
            if not isinstance(node, ast.Call):
                continue
            name = _is_native_call(node)
            if name is None:
                continue
            positional = [a for a in node.args if not isinstance(a, ast.Starred)]
            calls.append({
                "file": f"src/risa_attention/{path.name}",
                "line": node.lineno,
                "entry_point": name,
                "positional": len(positional),
                "positional_capsules": [i for i, a in enumerate(positional) if _wrapped(a)],
                "star_args": any(isinstance(a, ast.Starred) for a in node.args),
                "keywords": [k.arg for k in node.keywords if k.arg is not None],
                "keyword_capsules": [k.arg for k in node.keywords
                                     if k.arg is not None and _wrapped(k.value)],
                "star_kwargs": any(k.arg is None for k in node.keywords),
            })
    return calls


if __name__ == "__main__":
    reference = Path(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
    out = Path(__file__).resolve().parent / "reference_native_calls.json"
    out.write_text(json.dumps(extract(reference), indent=1) + "\n")
    print(f"{out}: {len(extract(reference))} calls")
