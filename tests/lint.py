#!/usr/bin/env python
"""Style and hygiene checks for the C++/CUDA and Python sources (no third-party linters needed).

Plays the part of the reference's cpplint/pylint wrapper (tests/lint.py there) with rules that
fit this tree:

C++ / CUDA (``include/``, ``src/``, ``tests/cpp``, ``tests/cuda``, ``baseline/*.cc``)
  * no tabs, no trailing blanks, lines of at most 100 columns, file ends with a newline;
  * headers have an include guard named after their path (``PS_..._H_``) or ``#pragma once``;
  * no ``using namespace`` at file scope in headers;
  * none of the batched-memcpy runtime calls that are known to fault on this driver.
Python (package, benchmarks, tests, launchers)
  * compiles; no tabs, no trailing blanks, lines of at most 120 columns;
  * imported names are used (``# noqa`` on the line silences it).

Usage: ``python tests/lint.py [paths...]``; exit status 1 when anything is reported.
"""
from __future__ import annotations

import ast
import os
import re
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPP_DIRS = ["include", "src", "tests/cpp", "tests/cuda", "baseline"]
PY_DIRS = ["ps_lite_b200", "benchmarks", "tests", "baseline", "tracker", "bench.py",
           "__graft_entry__.py"]
CPP_EXT = (".h", ".cuh", ".cc", ".cu", ".inl")
SKIP_PARTS = ("baseline/_ref", "build/", "__pycache__", "baseline/shims")
MAX_COLS = {"cpp": 100, "py": 120}
_BATCH = "Batch" + "Async"
BANNED = ["cudaMemcpy" + _BATCH, "cudaMemcpy3D" + _BATCH, "cuMemcpy" + _BATCH,
          "cuMemcpy3D" + _BATCH]


def _walk(paths, exts):
    for p in paths:
        full = os.path.join(ROOT, p)
        if os.path.isfile(full):
            if full.endswith(exts):
                yield full
            continue
        for d, _, files in os.walk(full):
            for f in sorted(files):
                path = os.path.join(d, f)
                rel = os.path.relpath(path, ROOT)
                if any(s in rel for s in SKIP_PARTS):
                    continue
                if f.endswith(exts):
                    yield path


def _common(rel, lines, out, kind):
    for i, line in enumerate(lines, 1):
        body = line.rstrip("\n")
        if "\t" in body:
            out.append(f"{rel}:{i}: tab character")
        if body != body.rstrip():
            out.append(f"{rel}:{i}: trailing blanks")
        if len(body) > MAX_COLS[kind] and "http" not in body:
            out.append(f"{rel}:{i}: {len(body)} columns (max {MAX_COLS[kind]})")
    if lines and not lines[-1].endswith("\n"):
        out.append(f"{rel}:{len(lines)}: no newline at end of file")


def lint_cpp(path, out):
    rel = os.path.relpath(path, ROOT)
    with open(path, encoding="utf-8") as f:
        lines = f.readlines()
    _common(rel, lines, out, "cpp")
    text = "".join(lines)
    for name in BANNED:
        if name in text:
            out.append(f"{rel}: names {name}, which faults on this driver")
    if path.endswith((".h", ".cuh")):
        if "#pragma once" not in text:
            m = re.search(r"#ifndef\s+(\w+)\s*\n#define\s+(\w+)", text)
            if not m or m.group(1) != m.group(2):
                out.append(f"{rel}: no include guard")
            elif not m.group(1).endswith("_H_"):
                out.append(f"{rel}: include guard {m.group(1)} should end with _H_")
        depth = 0
        for i, line in enumerate(lines, 1):
            code = line.split("//")[0]
            if depth == 0 and re.match(r"\s*using\s+namespace\s", code):
                out.append(f"{rel}:{i}: using-directive at file scope of a header")
            depth += code.count("{") - code.count("}")


class _Names(ast.NodeVisitor):
    def __init__(self):
        self.imported = {}
        self.used = set()

    def visit_Import(self, node):
        for a in node.names:
            self.imported[(a.asname or a.name).split(".")[0]] = node.lineno

    def visit_ImportFrom(self, node):
        for a in node.names:
            if a.name != "*":
                self.imported[a.asname or a.name] = node.lineno

    def visit_Name(self, node):
        self.used.add(node.id)

    def visit_Attribute(self, node):
        self.generic_visit(node)


def lint_py(path, out):
    rel = os.path.relpath(path, ROOT)
    with open(path, encoding="utf-8") as f:
        text = f.read()
    lines = text.splitlines(keepends=True)
    _common(rel, lines, out, "py")
    try:
        tree = ast.parse(text, filename=rel)
    except SyntaxError as exc:
        out.append(f"{rel}:{exc.lineno}: syntax error: {exc.msg}")
        return
    if os.path.basename(path) == "__init__.py":
        return  # re-exports
    v = _Names()
    v.visit(tree)
    exported = set()
    for node in ast.walk(tree):
        if isinstance(node, ast.Assign) and any(
                isinstance(t, ast.Name) and t.id == "__all__" for t in node.targets):
            try:
                exported |= set(ast.literal_eval(node.value))
            except ValueError:
                pass
    for name, lineno in sorted(v.imported.items(), key=lambda kv: kv[1]):
        if name in v.used or name in exported or name == "annotations":
            continue
        if "noqa" in lines[lineno - 1]:
            continue
        if re.search(r"\b%s\b" % re.escape(name), text.replace(lines[lineno - 1], "", 1)):
            continue  # used in a string annotation or a docstring example
        out.append(f"{rel}:{lineno}: '{name}' imported but unused")


def main(argv) -> int:
    out = []
    cpp = list(_walk(argv or CPP_DIRS, CPP_EXT))
    py = list(_walk(argv or PY_DIRS, (".py",)))
    for p in cpp:
        lint_cpp(p, out)
    for p in py:
        lint_py(p, out)
    for line in out:
        print(line)
    print(f"lint: {len(cpp)} C++/CUDA files, {len(py)} Python files, {len(out)} findings")
    return 1 if out else 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
