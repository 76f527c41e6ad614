"""Static checks of the source tree with the standard library only (no network, no extra tools):

* every ``.py`` file parses, has no tab indentation, no trailing white space and no line over
  110 columns;
* imports that a module never uses (names bound by ``import`` / ``from ... import`` that appear
  nowhere else in the file and are not re-exported through ``__all__`` or an ``__init__.py``);
* comments and docstrings do not point at files or tools that a reader of the sources does
  not have (build notes, one machine's paths).

    python ci/lint.py            # exit code 1 when something is found

The reference's lint step runs black, pylint and a licence-header check
(ci/task_lint.sh:9-21); this is the equivalent that runs on an offline machine.
"""
from __future__ import annotations

import ast
import os
import re
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SKIP_DIRS = {".git", "_work", "gpurun_out", "baseline/_ref", "__pycache__", ".pytest_cache",
             "slapo_b200/csrc/build"}
MAX_COLS = 110
FORBIDDEN = re.compile(r"SURVEY\.md|DESIGN\.md|VERDICT\.md|ADVICE\.md|BASELINE\.md|gpurun|/root/")
SOURCE_EXT = (".py", ".cu", ".cuh", ".cpp", ".h", ".sh")


def files():
    for base, dirs, names in os.walk(ROOT):
        rel = os.path.relpath(base, ROOT)
        dirs[:] = [d for d in dirs
                   if os.path.normpath(os.path.join(rel, d)) not in SKIP_DIRS and d not in SKIP_DIRS]
        for name in names:
            if name.endswith(SOURCE_EXT):
                yield os.path.join(base, name)


def unused_imports(tree, text, is_init):
    if is_init:
        return []
    bound = {}
    for node in ast.walk(tree):
        if isinstance(node, ast.Import):
            for a in node.names:
                bound[(a.asname or a.name).split(".")[0]] = node.lineno
        elif isinstance(node, ast.ImportFrom):
            for a in node.names:
                if a.name != "*":
                    bound[a.asname or a.name] = node.lineno
    used = {n.id for n in ast.walk(tree) if isinstance(n, ast.Name)}
    used |= {n.value.id for n in ast.walk(tree)
             if isinstance(n, ast.Attribute) and isinstance(n.value, ast.Name)}
    exported = set(re.findall(r"[\"']([A-Za-z_][A-Za-z0-9_]*)[\"']", text))   # __all__, strings
    lines = text.splitlines()
    out = []
    for name, line in bound.items():
        if name in used or name in exported or name == "annotations":
            continue
        if "noqa" in lines[line - 1]:
            continue
        out.append((line, f"'{name}' imported but unused"))
    return out


def main():
    problems = []
    for path in sorted(files()):
        rel = os.path.relpath(path, ROOT)
        if rel in ("ci/lint.py", "bench.py", "__graft_entry__.py"):
            policy = False     # these name the tools they are driven by
        else:
            policy = True
        with open(path, encoding="utf-8") as fh:
            text = fh.read()
        for i, line in enumerate(text.splitlines(), 1):
            if path.endswith(".py"):
                if line != line.rstrip():
                    problems.append((rel, i, "trailing white space"))
                if line.startswith("\t"):
                    problems.append((rel, i, "tab indentation"))
                if len(line) > MAX_COLS:
                    problems.append((rel, i, f"line longer than {MAX_COLS} columns"))
            if policy and FORBIDDEN.search(line):
                problems.append((rel, i, "points at a file / tool / path outside the sources"))
        if path.endswith(".py"):
            try:
                tree = ast.parse(text, filename=rel)
            except SyntaxError as err:
                problems.append((rel, err.lineno or 0, f"syntax error: {err.msg}"))
                continue
            for line, msg in unused_imports(tree, text, os.path.basename(path) == "__init__.py"):
                problems.append((rel, line, msg))
    for rel, line, msg in problems:
        print(f"{rel}:{line}: {msg}")
    print(f"{len(problems)} problem(s)")
    return 1 if problems else 0


if __name__ == "__main__":
    sys.exit(main())
