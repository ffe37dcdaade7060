"""Runs one of the reference's own test scripts (test/infiniop/<operator>.py, staged verbatim under
oracle/_ref/test_infiniop/ by oracle/build_ref.py) against whatever library $INFINI_ROOT names - in the tests,
this library.

    INFINI_ROOT=infinicore_b200 python tests/ref_harness.py paged_attention.py --nvidia

The scripts and the harness package beside them (libinfiniop/) run unmodified.  The one thing that has to give:
at import the harness sets argument types on the entry points of every operator the reference has (about 180),
and a library that carries only this path does not export the others.  The reference's maintainers would skip
the missing ones in op_register.py; here the same is done from outside, before the package's own __init__ runs:
OpRegister.register_lib is replaced by one that ignores the AttributeError of an operator the library lacks.
"""
import importlib.util
import runpy
import sys
import types
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
HARNESS = ROOT / "oracle" / "_ref" / "test_infiniop"


def load_tolerant_harness():
    pkg_dir = HARNESS / "libinfiniop"
    # a stand-in for the package, so that its submodules can be imported before its __init__ has run
    pkg = types.ModuleType("libinfiniop")
    pkg.__path__ = [str(pkg_dir)]
    pkg.__file__ = str(pkg_dir / "__init__.py")
    pkg.__package__ = "libinfiniop"
    sys.modules["libinfiniop"] = pkg
    sys.path.insert(0, str(HARNESS))
    sys.path.insert(0, str(pkg_dir))  # the package's __init__ does the same

    op_register = importlib.import_module("libinfiniop.op_register")
    skipped = []

    def register_lib(lib, registry=op_register.OpRegister.registry):
        for op in registry:
            try:
                op(lib)
            except AttributeError:
                skipped.append(op.__name__)

    op_register.OpRegister.register_lib = staticmethod(register_lib)

    # now the package's own __init__, in the stand-in's namespace (it imports liboperators, which opens the
    # libraries under $INFINI_ROOT/lib and registers the operators)
    spec = importlib.util.spec_from_file_location("libinfiniop", pkg_dir / "__init__.py", submodule_search_locations=[str(pkg_dir)])
    pkg.__spec__ = spec
    spec.loader.exec_module(pkg)
    return skipped


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    script = HARNESS / sys.argv[1]
    if not script.is_file():
        raise SystemExit(f"{script} is not staged: run `python -m oracle.build_ref` where the reference checkout is")
    skipped = load_tolerant_harness()
    print(f"[ref_harness] {len(skipped)} operators of the reference are not in this library and were skipped at registration", flush=True)
    sys.argv = [str(script)] + sys.argv[2:]
    runpy.run_path(str(script), run_name="__main__")


if __name__ == "__main__":
    main()
