"""The bench's workload table and the runners behind it agree (no GPU needed): every workload name the default line's
`paths` record runs has a runner, the module docstring describes it, and the product never imports the oracle."""
import ast
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _module_constants(path, names):
    tree = ast.parse(open(path).read())
    out = {}
    for node in tree.body:
        if isinstance(node, ast.Assign) and len(node.targets) == 1 and isinstance(node.targets[0], ast.Name):
            if node.targets[0].id in names:
                out[node.targets[0].id] = node.value
    return tree, out


def test_every_path_workload_has_a_runner_and_a_description():
    _, bench = _module_constants(os.path.join(ROOT, "bench.py"), {"PATH_WORKLOADS"})
    workloads = [elt.value for elt in bench["PATH_WORKLOADS"].elts]
    tree, paths = _module_constants(os.path.join(ROOT, "bench_paths.py"), {"RUNNERS"})
    runners = {k.value: v.id for k, v in zip(paths["RUNNERS"].keys, paths["RUNNERS"].values)}
    defined = {n.name for n in tree.body if isinstance(n, ast.FunctionDef)}
    doc = ast.get_docstring(tree)
    assert sorted(workloads) == sorted(runners), "bench.py and bench_paths.py list different workloads"
    for name in workloads:
        assert runners[name] in defined, f"{name}: runner {runners[name]} is not defined"
        assert name in doc, f"{name} is not described in bench_paths.py's docstring"


def test_the_package_never_touches_the_oracle():
    pkg = os.path.join(ROOT, "itak_torch_rebuild_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".hpp", ".h")):
                text = open(os.path.join(dirpath, f), errors="replace").read()
                assert "oracle" not in text.lower() or f == "build.py", f"{f} mentions the oracle"
