"""Repository rules that can be checked without a GPU."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _py_files(folder):
    for base, _, names in os.walk(os.path.join(ROOT, folder)):
        for n in names:
            if n.endswith(".py"):
                yield os.path.join(base, n)


def test_the_package_never_touches_the_oracle():
    """The oracle is the checker: nothing under flame_b200/ may import, load or execute it."""
    for path in _py_files("flame_b200"):
        text = open(path).read()
        assert not re.search(r"^\s*(from|import)\s+oracle\b", text, re.M), path
        assert "liboracle" not in text and "oracle/" not in text, path
    for name in os.listdir(os.path.join(ROOT, "flame_b200", "csrc")):
        if name.endswith((".cu", ".cuh", ".h", "Makefile")):
            assert "oracle" not in open(os.path.join(ROOT, "flame_b200", "csrc", name)).read().lower(), name


def test_bench_uses_the_oracle_only_as_checker_and_cpu_baseline():
    """bench.py may use the oracle to check results after a timed region, as the reported CPU baseline and in the
    reference arm; never inside the product's timed path.  Which functions import it is fixed here."""
    import ast

    tree = ast.parse(open(os.path.join(ROOT, "bench.py")).read())
    users, callers = set(), set()
    for fn in ast.walk(tree):
        if not isinstance(fn, ast.FunctionDef):
            continue
        for node in ast.walk(fn):
            if isinstance(node, ast.ImportFrom) and (node.module or "").split(".")[0] == "oracle":
                users.add(fn.name)
            if isinstance(node, ast.Import) and any(a.name.split(".")[0] == "oracle" for a in node.names):
                users.add(fn.name)
            if isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and node.func.id == "reference_gpu_path":
                callers.add(fn.name)
    # checkers (run after the timed loops), the CPU baseline, and the reference arm's own GPU path
    assert users <= {"verify_against_oracle", "verify_restored", "run_fp8_mixed", "run_weight_stream", "cpu_leg", "reference_gpu_path"}, users
    assert not any(isinstance(n, (ast.Import, ast.ImportFrom)) and "oracle" in ast.dump(n) for n in tree.body), "no module-level import of the oracle"
    # the compiled reference files are timed by the --impl reference arm only, never by this library's arm
    assert callers == {"run_reference_arm"}, callers


def _ignored_top_level_folders():
    """Top-level folders that .gitignore keeps out of the history (working files, run output, build output)."""
    out = []
    for line in open(os.path.join(ROOT, ".gitignore")):
        line = line.strip()
        if line.endswith("/") and not line.startswith("#") and "*" not in line:
            name = line.strip("/")
            if "/" not in name and not name.startswith(".") and name not in ("build", "__pycache__"):
                out.append(name)
    return out


def test_nothing_committed_reads_a_folder_that_is_not_committed():
    """Working files and run output are not part of the product: no committed Python file may name their folders in a
    path.  (The compiled reference under oracle/ is named by oracle/ itself, which builds it.)"""
    folders = _ignored_top_level_folders()
    assert folders, "expected .gitignore to list the working folder"
    pattern = re.compile(r"[\"'/](" + "|".join(re.escape(f) for f in folders) + r")/")
    allowed_output = {f for f in folders if f.endswith("_out")}      # a folder that only receives what a run writes
    for folder in ("flame_b200", "tests", "oracle"):
        for path in _py_files(folder):
            if path.endswith("test_layout_rules.py"):
                continue
            hits = {m.group(1) for m in pattern.finditer(open(path).read())} - allowed_output
            assert not hits, (path, hits)
    for name in ("bench.py", "__graft_entry__.py"):
        hits = {m.group(1) for m in pattern.finditer(open(os.path.join(ROOT, name)).read())} - allowed_output
        assert not hits, (name, hits)


def test_no_committed_source_holds_an_absolute_home_path():
    """Paths of the machine a file was written on do not belong in it: the reference checkout, where one exists, is
    found through the REF make variable or the FLAME_REFERENCE_DIR environment variable."""
    home = os.path.expanduser("~")
    if len(home) < 4:
        return
    for folder in ("flame_b200", "tests", "oracle", "include"):
        for base, _, names in os.walk(os.path.join(ROOT, folder)):
            if "_ref" in base or "__pycache__" in base:
                continue
            for n in names:
                if n.endswith((".py", ".c", ".cu", ".cuh", ".h", "Makefile")):
                    assert home + "/" not in open(os.path.join(base, n), errors="replace").read(), os.path.join(base, n)
    for name in ("bench.py", "__graft_entry__.py"):
        assert home + "/" not in open(os.path.join(ROOT, name)).read(), name


def test_kernels_are_built_with_ieee_semantics():
    mk = open(os.path.join(ROOT, "flame_b200", "csrc", "Makefile")).read()
    flags = "\n".join(l for l in mk.splitlines() if not l.lstrip().startswith("#"))
    assert "use_fast_math" not in flags and "-ftz=true" not in flags
    assert "compute_100a,code=sm_100a" in flags
