"""Static check that runs without a GPU: every call of a native op (``lib.<op>(...)`` / ``native.lib().<op>(...)``)
in the package, the tests and the benchmark names an op the library registers and passes a number of arguments
that op's schema accepts.  The ops themselves only run on a GPU, so a binding that drifted from its call sites
would otherwise first show on a GPU box."""
import ast
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def _is_lib_call(base: ast.AST) -> bool:
    if isinstance(base, ast.Name):
        return base.id == "lib"
    if isinstance(base, ast.Call):
        f = base.func
        return (isinstance(f, ast.Attribute) and f.attr == "lib") or (isinstance(f, ast.Name) and f.id == "lib")
    return False


def test_native_op_call_sites_match_the_registered_schemas():
    from piper_b200.ops import native

    if not native.lib_path().exists():
        pytest.skip("the native library has not been built")
    torch.ops.load_library(str(native.lib_path()))
    ns = torch.ops.piper_c
    files = sorted((ROOT / "piper_b200").rglob("*.py")) + sorted((ROOT / "tests").glob("*.py")) \
        + [ROOT / "bench.py", ROOT / "__graft_entry__.py"]
    problems, checked = [], 0
    for path in files:
        for node in ast.walk(ast.parse(path.read_text())):
            if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and _is_lib_call(node.func.value)):
                continue
            if any(isinstance(a, ast.Starred) for a in node.args):
                continue
            name = node.func.attr
            op = getattr(ns, name, None)
            if op is None:
                problems.append(f"{path.relative_to(ROOT)}:{node.lineno}: no native op named {name}")
                continue
            args = op.default._schema.arguments
            required = sum(1 for a in args if not a.has_default_value())
            given = len(node.args) + len(node.keywords)
            checked += 1
            if not required <= given <= len(args):
                problems.append(f"{path.relative_to(ROOT)}:{node.lineno}: {name} gets {given} arguments, "
                                f"its schema takes {required}..{len(args)}")
    assert not problems, "\n".join(problems)
    assert checked > 100
