"""Build recipe for ``oracle/_ref``: the reference project's own CPU implementation of the path, compiled.

TEST/BENCH INFRASTRUCTURE, not product code.  The reference's CPU path is two pure-Python modules
(w4a16/quantization.py and w4a16/reference.py inside the reference project).  Where a checkout of the
reference is present, this recipe byte-compiles those two files *from where they lie* into
``oracle/_ref/w4a16/*.bin`` (CPython code objects in the ``.pyc`` container; the suffix is not ``.pyc``
because tools that copy a working tree commonly leave ``*.pyc`` behind) -- compiled outputs only; no
reference source enters this repository.  ``load()`` installs them as the modules ``w4a16``,
``w4a16.quantization`` and ``w4a16.reference`` of the calling interpreter, which must not have imported
another package called ``w4a16``.  ``oracle/_ref`` is ignored by git and travels with the working tree, so the benchmark's reference arm (``bench.py --impl reference``) and its ``cpu_baseline`` leg can
time the reference itself on a machine that has no checkout; without it they time the restatement in
``oracle/torch_cpu_port.py`` and say so (``kind: "port"``).

    python oracle/build_ref.py [/path/to/reference]
"""
from __future__ import annotations

import pathlib
import py_compile
import sys

HERE = pathlib.Path(__file__).resolve().parent
OUT = HERE / "_ref" / "w4a16"
MODULES = ("quantization", "reference")
DEFAULT_CHECKOUT = pathlib.Path("/root/reference")


def build(checkout: pathlib.Path = DEFAULT_CHECKOUT) -> bool:
    """Compile the reference's CPU modules into oracle/_ref; False when there is no checkout."""
    sources = [checkout / "w4a16" / f"{name}.py" for name in MODULES]
    if not all(source.is_file() for source in sources):
        return False
    OUT.mkdir(parents=True, exist_ok=True)
    for name, source in zip(MODULES, sources):
        py_compile.compile(str(source), cfile=str(OUT / f"{name}.bin"), dfile=f"<reference>/w4a16/{name}.py", doraise=True)
    return True


def available() -> bool:
    return all((OUT / f"{name}.bin").is_file() for name in MODULES)


def load():
    """Install the compiled reference modules in this interpreter; returns (quantization, reference)."""
    import importlib.machinery
    import importlib.util
    import types

    if not available():
        raise ImportError("oracle/_ref is not built: run oracle/build_ref.py where a checkout of the reference exists")
    if "w4a16" in sys.modules and getattr(sys.modules["w4a16"], "__path__", None) != [str(OUT)]:
        raise ImportError("another package called w4a16 is already imported in this interpreter")
    package = types.ModuleType("w4a16")
    package.__path__ = [str(OUT)]
    sys.modules["w4a16"] = package
    loaded = []
    for name in MODULES:
        full = f"w4a16.{name}"
        loader = importlib.machinery.SourcelessFileLoader(full, str(OUT / f"{name}.bin"))
        spec = importlib.util.spec_from_loader(full, loader)
        module = importlib.util.module_from_spec(spec)
        sys.modules[full] = module
        loader.exec_module(module)
        setattr(package, name, module)
        loaded.append(module)
    return tuple(loaded)


if __name__ == "__main__":
    ok = build(pathlib.Path(sys.argv[1]) if len(sys.argv) > 1 else DEFAULT_CHECKOUT)
    print("oracle/_ref built" if ok else "no reference checkout: oracle/_ref not built")
