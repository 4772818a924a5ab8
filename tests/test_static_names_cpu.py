"""Static check for names that are referenced but defined nowhere (module scope, enclosing scopes, builtins).

Most GPU-only branches (peer-memory back ends, CUDA bindings, the benchmark's reference arm) never execute in the CPU
suite, so a misspelt or stale name there would only surface on a GPU box; ``symtable`` finds them without running."""
import builtins
import os
import symtable

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _undefined_in(path):
    with open(path) as f:
        src = f.read()
    top = symtable.symtable(src, path, "exec")
    module_names = {s.get_name() for s in top.get_symbols() if s.is_assigned() or s.is_imported() or s.is_namespace()}
    if "*" in src and "import *" in src:
        return []
    bad = [f"{os.path.relpath(path, ROOT)}:<module>:{s.get_name()}" for s in top.get_symbols()
           if s.is_referenced() and not (s.is_assigned() or s.is_imported() or s.is_namespace())
           and not hasattr(builtins, s.get_name()) and s.get_name() not in ("__file__", "__name__", "__doc__")]

    def walk(table):
        for child in table.get_children():
            if child.get_type() in ("function", "class"):
                for s in child.get_symbols():
                    if s.is_global() and s.is_referenced() and not s.is_assigned():
                        n = s.get_name()
                        if n not in module_names and not hasattr(builtins, n) and n not in ("__file__", "__name__", "__doc__"):
                            bad.append(f"{os.path.relpath(path, ROOT)}:{child.get_name()}:{n}")
            walk(child)

    walk(top)
    return bad


def test_no_undefined_names_in_sources():
    files = [os.path.join(ROOT, f) for f in ("bench.py", "train.py", "download.py", "__graft_entry__.py")]
    for base in ("flextrain_b200", "baseline/baseline_harness", "baseline/scripts", "baseline/backends", "experiments",
                 "examples", "tests"):
        for d, _, names in os.walk(os.path.join(ROOT, base)):
            files += [os.path.join(d, n) for n in names if n.endswith(".py")]
    files.append(os.path.join(ROOT, "baseline", "run_baseline.py"))
    bad = []
    for f in sorted(set(files)):
        if os.path.exists(f):
            bad += _undefined_in(f)
    assert not bad, "undefined names: " + ", ".join(bad)
