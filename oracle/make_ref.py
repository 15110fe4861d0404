"""Build ``oracle/_ref``: the UNMODIFIED reference implementation as test infrastructure.

    python oracle/make_ref.py [--reference /path/to/BiBo-checkout]

The reference is pure Python, so "building" it means byte-compiling its ``src`` package
(configuration, model, attention, feed-forward, router: nineteen files) into sourceless ``.pyc``
modules, packed into ONE archive ``oracle/_ref/reference_src.zip`` (``activate()`` unpacks it into a
temporary directory and imports from there).  No source file is copied; the directory is git-ignored and is never imported by the
product (``bibo_b200``): only tests, ``__graft_entry__`` and ``bench.py``'s reference legs put the
archive on ``sys.path``.  With it a machine without the checkout can still

* run the reference's own ``BiBoModel`` / ``BiBoMoELayer`` as the checker of the whole-model tests, and
* time the reference's eager MoE layer on the CPU and on the GPU next to the kernels.

The ``.pyc`` files are tied to the interpreter version that wrote them (``sys.implementation.cache_tag``
is recorded in ``oracle/_ref/BUILD_INFO``); ``available()`` refuses a mismatch.
"""
from __future__ import annotations

import argparse
import os
import pathlib
import py_compile
import shutil
import sys
import tempfile
import zipfile

HERE = pathlib.Path(__file__).resolve().parent
OUT = HERE / "_ref"
ARCHIVE = OUT / "reference_src.zip"
DEFAULT_REFERENCE = os.environ.get("BIBO_REFERENCE", "/root/reference")


def build(reference: str = DEFAULT_REFERENCE, quiet: bool = False) -> pathlib.Path:
    src = pathlib.Path(reference) / "src"
    if not src.is_dir():
        raise FileNotFoundError(f"{src} not found: point --reference at a checkout of the reference")
    if OUT.exists():
        shutil.rmtree(OUT)
    OUT.mkdir(parents=True)
    n = 0
    with tempfile.TemporaryDirectory() as tmp, zipfile.ZipFile(ARCHIVE, "w", zipfile.ZIP_DEFLATED) as zf:
        for py in sorted(src.rglob("*.py")):
            rel = py.relative_to(src.parent)
            target = (pathlib.Path(tmp) / rel).with_suffix(".pyc")
            target.parent.mkdir(parents=True, exist_ok=True)
            # dfile: what tracebacks show (the file's path inside its project), not a path of this machine
            py_compile.compile(str(py), cfile=str(target), dfile=str(rel), doraise=True,
                               invalidation_mode=py_compile.PycInvalidationMode.UNCHECKED_HASH)
            zf.write(target, str(rel.with_suffix(".pyc")))
            n += 1
    (OUT / "BUILD_INFO").write_text(f"{sys.implementation.cache_tag}\n{n} modules\n")
    if not quiet:
        print(f"{OUT}: {n} modules byte-compiled ({sys.implementation.cache_tag})")
    return OUT


def available() -> bool:
    info = OUT / "BUILD_INFO"
    return ARCHIVE.exists() and info.exists() and info.read_text().split("\n")[0] == sys.implementation.cache_tag


_unpacked = None


def activate() -> None:
    """Make the compiled reference importable (its top-level package is ``src``): the archive is unpacked into
    a temporary directory of this process, removed at exit, and that directory goes on ``sys.path`` (a model
    class of the reference wants a real file behind its module, which an archive member is not)."""
    global _unpacked
    if not available():
        raise RuntimeError("oracle/_ref is missing or was built by another Python: run `python oracle/make_ref.py`")
    if _unpacked is None:
        import atexit
        _unpacked = tempfile.mkdtemp(prefix="bibo_ref_")
        atexit.register(shutil.rmtree, _unpacked, ignore_errors=True)
        with zipfile.ZipFile(ARCHIVE) as zf:
            zf.extractall(_unpacked)
    if _unpacked not in sys.path:
        sys.path.insert(0, _unpacked)
    os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    build(ap.parse_args().reference)
