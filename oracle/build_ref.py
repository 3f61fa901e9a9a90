"""Build ``oracle/_ref/``: the UNMODIFIED reference, byte-compiled where it lies.  TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref.py [--reference /path/to/WorkloadSuite]

The reference is pure Python, so "building" it means compiling two of its files to
CPython bytecode -- no source is copied, nothing is edited:

* ``workloads/mamba/model_ref.py`` -> ``oracle/_ref/model_ref.bc``  (``SSDLayer._ssd_core``,
  ``model_ref.py:123-162``, and the whole ``Model``, ``:165-229``),
* ``bench.py``                      -> ``oracle/_ref/ref_bench.bc``  (the reference's timing
  harness, ``bench.py:138-268``).

(The files are ordinary ``.pyc`` images under another suffix: tools that copy a working copy
between machines tend to drop ``*.pyc`` as caches.)

``oracle/_ref/`` is git-ignored build output (like the package's ``.so``); it travels with a
working copy to a machine that has no reference checkout.  ``load_model_ref()`` /
``load_ref_bench()`` import the bytecode with ``SourcelessFileLoader``; they return ``None`` when
the directory was never built (the callers then fall back to the oracle's restatement and say
so).  Only the benchmark's CPU-reference legs and the tests use this module; the product
package never does.
"""
from __future__ import annotations

import argparse
import importlib.machinery
import importlib.util
import json
import py_compile
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
DEFAULT_REFERENCE = Path("/root/reference")

_FILES = {
    "model_ref.bc": Path("workloads") / "mamba" / "model_ref.py",
    "ref_bench.bc": Path("bench.py"),
}


def build(reference: Path = DEFAULT_REFERENCE, quiet: bool = True) -> bool:
    """Compile the reference's files into ``oracle/_ref``.  Returns False (and builds nothing)
    when there is no reference checkout at ``reference``."""
    reference = Path(reference)
    if not all((reference / rel).is_file() for rel in _FILES.values()):
        return False
    REF_DIR.mkdir(exist_ok=True)
    for out, rel in _FILES.items():
        # dfile: the path shown in tracebacks is the file's path inside the reference project
        py_compile.compile(str(reference / rel), cfile=str(REF_DIR / out), dfile=str(rel), doraise=True,
                           invalidation_mode=py_compile.PycInvalidationMode.UNCHECKED_HASH)
    (REF_DIR / "BUILT_FROM.json").write_text(json.dumps({
        "python": sys.version.split()[0], "files": {k: str(v) for k, v in _FILES.items()},
        "how": "py_compile of the unmodified reference files; no source copied"}, indent=1))
    if not quiet:
        print(f"built {REF_DIR}")
    return True


def _load(pyc: str, name: str):
    path = REF_DIR / pyc
    if not path.is_file():
        return None
    if name in sys.modules:
        return sys.modules[name]
    loader = importlib.machinery.SourcelessFileLoader(name, str(path))
    spec = importlib.util.spec_from_loader(name, loader)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    try:
        loader.exec_module(mod)
    except Exception:
        sys.modules.pop(name, None)
        raise
    return mod


def load_model_ref():
    """The reference's ``workloads/mamba/model_ref.py`` as a module, or None if ``_ref`` is not built."""
    return _load("model_ref.bc", "ws_mamba_model_ref")


def load_ref_bench():
    """The reference's ``bench.py`` as a module (nothing runs at import), or None."""
    return _load("ref_bench.bc", "ws_reference_bench")


def reference_core(mod, X, A, B, C, chunk, dt=None):
    """Call the unmodified ``SSDLayer._ssd_core`` (``model_ref.py:123-162``) on un-chunked tensors.

    X [b,s,h,p] fp16, A [b,s,h] fp32 log-decay, B/C [b,s,h,n] fp16 already broadcast to heads (the caller
    does that outside any timed region, as ``SSDLayer.forward`` does at ``model_ref.py:97-99``),
    dt [b,s,h] fp16 or None (ones).  Returns Y [b,s,h,p] fp16."""
    import torch

    b, s, h, p = X.shape
    n = B.shape[-1]
    c = s // chunk
    key = (h, n, p, chunk)
    cache = reference_core.__dict__.setdefault("_layers", {})
    layer = cache.get(key)
    if layer is None:
        # _ssd_core reads only block_len, n_heads, d_state and d_head of the layer (model_ref.py:140,153); a
        # narrow d_model keeps the unused projections small
        layer = mod.SSDLayer(d_model=64, n_heads=h, d_state=n, d_head=p, n_groups=1, block_len=chunk)
        cache[key] = layer
    if dt is None:
        dt = torch.ones(b, s, h, dtype=X.dtype)
    Y = layer._ssd_core(X.reshape(b, c, chunk, h, p), B.reshape(b, c, chunk, h, n), C.reshape(b, c, chunk, h, n),
                        dt.reshape(b, c, chunk, h), A.reshape(b, c, chunk, h), b)
    return Y.reshape(b, s, h, p)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=str(DEFAULT_REFERENCE))
    a = ap.parse_args()
    ok = build(Path(a.reference), quiet=False)
    if not ok:
        print(f"no reference checkout at {a.reference}: nothing built")
