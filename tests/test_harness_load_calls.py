"""CPU tier: every `load(...)` call that the reference harnesses make, read from a reference checkout as text
and passed to the stand-in literally (same keyword arguments, same flag lists).  The harness files are only
parsed: module-level constants are evaluated to resolve the arguments, nothing else of them runs.  Skipped
when no checkout is found (argument-free discovery as in oracle/build_ref.py: $RWKV_CUDA_REF, baseline/_ref,
a sibling directory `reference`)."""
import ast
import os

import pytest
import torch

import rwkv_cuda_b200 as R
from oracle import build_ref

HARNESSES = ["wkv/run.py", "depthwise_conv1d/run.py", "wkv5/run.py", "wkv5_bf16/run.py", "wkv5a/run.py", "wkv6/run.py",
             "wkv6_state/run.py", "rwkv7_fast_fused/rwkv7_cuda_benchmark.py",
             "rwkv7_fast_fused/rwkv7_cuda_benchmark_state.py",
             "rwkv7_fast_fused/rwkv7_cuda_benchmark_state_passing.py"]
KNOWN = {"wkv", "timex", "wkv5", "wkv5a", "wkv6", "wkv6state", "rwkv7_clampw", "rwkv7_state_clampw",
         "rwkv7_statepassing_clampw"}


class _Argv:
    """Stands in for `sys` while the constants are evaluated: the harnesses read their mode from argv."""
    argv = ["harness.py", "bf16", "0", "0"]


def _is_constant_expression(node):
    """No call other than conversions and string methods: tensors, file and device access are left alone."""
    for n in ast.walk(node):
        if isinstance(n, ast.Call):
            f = n.func
            ok = (isinstance(f, ast.Name) and f.id in ("int", "float", "str", "len", "min", "max")) or \
                 (isinstance(f, ast.Attribute) and f.attr in ("strip", "replace", "lower"))
            if not ok:
                return False
    return True


def _load_calls(path):
    """(keyword arguments) of every load(...) call of a harness, resolved against the constants that the
    harness assigns before the call (in file order, any nesting)."""
    tree = ast.parse(open(path).read())
    env = {"torch": torch, "os": os, "sys": _Argv}
    calls = []

    def visit(node):
        for child in ast.iter_child_nodes(node):
            if isinstance(child, ast.Assign) and _is_constant_expression(child.value):
                try:
                    exec(compile(ast.Module([child], []), path, "exec"), env)   # noqa: S102 (a constant of a harness)
                except Exception:
                    pass
            for call in [n for n in ast.walk(child) if isinstance(child, (ast.Assign, ast.Expr)) and isinstance(n, ast.Call)]:
                fn = call.func
                if (isinstance(fn, ast.Name) and fn.id == "load") or (isinstance(fn, ast.Attribute) and fn.attr == "load"
                                                                      and "cpp_extension" in ast.unparse(fn)):
                    kw = {}
                    for k in call.keywords:
                        kw[k.arg] = eval(compile(ast.Expression(k.value), path, "eval"), env)
                    calls.append(kw)
            if not isinstance(child, (ast.Assign, ast.Expr)):
                visit(child)

    visit(tree)
    return calls


@pytest.mark.parametrize("harness", HARNESSES)
def test_reference_harness_load_calls_are_accepted(harness):
    ref = build_ref.checkout()
    if ref is None or not os.path.exists(os.path.join(ref, harness)):
        pytest.skip("no reference checkout with this harness")
    calls = _load_calls(os.path.join(ref, harness))
    assert calls, "the harness has no load(...) call"
    seen = 0
    for kw in calls:
        if kw["name"] not in KNOWN:       # wkv5/run.py also builds a second, older kernel of its own as a checker
            assert kw["name"].endswith("_ref")
            continue
        seen += 1
        mod = R.load(**kw)
        if kw.get("is_python_module", True):
            assert callable(mod.forward) and callable(mod.backward)
            flags = kw.get("extra_cuda_cflags", [])
            for f in flags:
                if f.startswith("-D_N_="):
                    assert mod.defines["_N_"] == int(f.split("=")[1])
        else:
            assert mod is None
            ns = getattr(torch.ops, kw["name"])
            assert ns.forward is not None and ns.backward is not None
    assert seen >= 1
