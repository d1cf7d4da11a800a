"""Static check of the Python host side: every name a function reads is bound somewhere it can see.

The package's GPU paths (handle methods, the bench's multi-rank reporting) cannot run on a machine without a GPU, so a
misspelt or never-imported name in them would first show on the GPU box. This test walks the syntax trees instead:
for every function, the names it loads must be builtins, module-level names, or names bound somewhere inside the
outermost function that contains it (arguments, assignments, imports, loop / with / except targets, nested
definitions). The binding analysis is flow-insensitive, so it reports no false alarms; it catches undefined names only.
"""
import ast
import builtins
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "test-model-thing-cuda_b200", "tmt_moe_b200")


def _bound_names(node):
    """Every name bound anywhere inside `node` (nested scopes included)."""
    out = set()
    for n in ast.walk(node):
        if isinstance(n, ast.Name) and isinstance(n.ctx, (ast.Store, ast.Del)):
            out.add(n.id)
        elif isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef)):
            out.add(n.name)
        elif isinstance(n, ast.arg):
            out.add(n.arg)
        elif isinstance(n, (ast.Import, ast.ImportFrom)):
            for a in n.names:
                out.add((a.asname or a.name).split(".")[0])
        elif isinstance(n, ast.ExceptHandler) and n.name:
            out.add(n.name)
        elif isinstance(n, (ast.Global, ast.Nonlocal)):
            out.update(n.names)
        elif isinstance(n, ast.MatchAs) and n.name:
            out.add(n.name)
    return out


def _level_names(stmts):
    """Names bound by these statements themselves, not inside a function or class body below them (conditional blocks count)."""
    out = set()
    for s in stmts:
        if isinstance(s, (ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef)):
            out.add(s.name)
            continue
        for n in ast.walk(s):
            if isinstance(n, ast.Name) and isinstance(n.ctx, ast.Store):
                out.add(n.id)
            elif isinstance(n, (ast.Import, ast.ImportFrom)):
                for a in n.names:
                    out.add((a.asname or a.name).split(".")[0])
            elif isinstance(n, ast.ExceptHandler) and n.name:
                out.add(n.name)
    return out


def _module_names(tree):
    out = _level_names(tree.body)
    for n in ast.walk(tree):            # names a function declares global and assigns
        if isinstance(n, ast.Global):
            out.update(n.names)
    return out


def undefined_names(path):
    tree = ast.parse(open(path).read(), path)
    known = set(dir(builtins)) | _module_names(tree) | {"__file__", "__name__", "__doc__"}
    bad = []

    def check_function(fn, extra):
        ok = known | extra | _bound_names(fn)
        for n in ast.walk(fn):
            if isinstance(n, ast.Name) and isinstance(n.ctx, ast.Load) and n.id not in ok:
                bad.append("%s:%d %s (in %s)" % (os.path.basename(path), n.lineno, n.id, fn.name))

    def visit(stmts, extra):
        for s in stmts:
            if isinstance(s, (ast.FunctionDef, ast.AsyncFunctionDef)):
                check_function(s, extra)
            elif isinstance(s, ast.ClassDef):
                visit(s.body, extra | _level_names(s.body))
            else:
                for n in ast.walk(s):
                    if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef)):
                        check_function(n, extra)
    visit(tree.body, set())
    return bad


def _host_files():
    files = [os.path.join(ROOT, "bench.py"), os.path.join(ROOT, "__graft_entry__.py")]
    for d in (PKG, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):
        files += sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(".py"))
    return files


@pytest.mark.parametrize("path", _host_files(), ids=lambda p: os.path.relpath(p, ROOT))
def test_no_undefined_names(path):
    assert undefined_names(path) == []


def test_the_check_sees_a_missing_import(tmp_path):
    p = tmp_path / "m.py"
    # another method's local import must not hide it
    p.write_text("import os\n\nclass A:\n    def g(self):\n        import numpy as np\n        return np\n\n"
                 "    def f(self):\n        import ctypes\n        return np.zeros(1), os.sep, ctypes\n")
    assert [b.split()[1] for b in undefined_names(str(p))] == ["np"]
