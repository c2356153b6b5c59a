"""Build recipe for ``oracle/_ref``: the reference project's own CPU implementation of the path, compiled.

TEST/BENCH INFRASTRUCTURE, not product code.  The reference's CPU path is two pure-Python modules
(w4a16/quantization.py and w4a16/reference.py inside the reference project).  Where a checkout of the
reference is present, this recipe byte-compiles those two files *from where they lie* into
``oracle/_ref/w4a16/*.pyc`` -- compiled outputs only; no reference source enters this repository -- next to
an empty package marker, so that ``import w4a16.reference`` resolves to the reference's code in a process
that puts ``oracle/_ref`` first on ``sys.path``.  ``oracle/_ref`` is ignored by git and travels with the
working tree, so the benchmark's reference arm (``bench.py --impl reference``) and its ``cpu_baseline`` leg can
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
    (OUT / "__init__.py").write_text('"""Compiled CPU modules of the reference project (see oracle/build_ref.py)."""\n')
    for name, source in zip(MODULES, sources):
        py_compile.compile(str(source), cfile=str(OUT / f"{name}.pyc"), dfile=f"<reference>/w4a16/{name}.py", doraise=True)
    return True


def available() -> bool:
    return all((OUT / f"{name}.pyc").is_file() for name in MODULES) and (OUT / "__init__.py").is_file()


if __name__ == "__main__":
    ok = build(pathlib.Path(sys.argv[1]) if len(sys.argv) > 1 else DEFAULT_CHECKOUT)
    print("oracle/_ref built" if ok else "no reference checkout: oracle/_ref not built")
