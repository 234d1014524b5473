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
    text = open(os.path.join(ROOT, "bench.py")).read()
    users = {m.group(1) for m in re.finditer(r"def (\w+)\([^)]*\):(?:(?!\ndef ).)*?from oracle import", text, re.S)}
    assert users <= {"verify_against_oracle", "cpu_leg", "reference_gpu_path"}, users
    # the compiled reference files are timed by the --impl reference arm only, never by this library's arm
    callers = {m.group(1) for m in re.finditer(r"def (\w+)\([^)]*\):(?:(?!\ndef ).)*?reference_gpu_path\(", text, re.S)}
    assert callers == {"run_reference_arm"}, callers


def test_nothing_committed_reads_the_working_folder_or_the_reference_checkout():
    for folder in ("flame_b200", "tests", "oracle"):
        for path in _py_files(folder):
            if path.endswith("test_layout_rules.py"):
                continue
            text = open(path).read()
            assert not re.search(r"[\"'/]_work/", text), path
            if not path.endswith(os.path.join("oracle", "capi.py")):
                assert "/root/reference" not in text, path
    for name in ("bench.py", "__graft_entry__.py"):
        text = open(os.path.join(ROOT, name)).read()
        assert not re.search(r"[\"'/]_work/", text) and "/root/reference" not in text, name


def test_kernels_are_built_with_ieee_semantics():
    mk = open(os.path.join(ROOT, "flame_b200", "csrc", "Makefile")).read()
    flags = "\n".join(l for l in mk.splitlines() if not l.lstrip().startswith("#"))
    assert "use_fast_math" not in flags and "-ftz=true" not in flags
    assert "compute_100a,code=sm_100a" in flags
