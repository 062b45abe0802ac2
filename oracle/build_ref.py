"""Installs the UNMODIFIED reference packages into ``oracle/_ref`` (TEST INFRASTRUCTURE ONLY).

The reference is pure Python (PyTorch + Triton): "building" it is a plain offline pip install
of its two source trees, the core package ``inquant`` and the vLLM extension ``inquant_vllm``,
from a scratch copy (the checkout is read-only and setuptools writes egg-info next to the
sources).  ``oracle/_ref`` is git-ignored, so no reference source enters the history, but it
travels with the built artefacts to the machine that runs the GPU legs.  Consumers:

* ``bench.py --impl reference`` times the reference's own torch CPU path from it;
* ``bench.py`` (CUDA arm, one GPU) runs the reference's Triton decode kernel from it beside this
  library's kernel on the same packed layer, and counts the packed bytes on which the
  reference's torch CUDA encoders and this library's encoders differ;
* nothing in the shipped package imports it.

The installed package is called ``inquant`` like this repository's mirror of it, so consumers
load it under another name with ``load_reference()``.

    python oracle/build_ref.py [/path/to/reference/checkout]
"""
from __future__ import annotations

import importlib.util
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")


def build(reference: str = "/root/reference") -> str | None:
    """pip-installs both reference packages into ``oracle/_ref``; returns the target or None when
    the checkout is absent (the target of an earlier build is then left as it is)."""
    if not os.path.isdir(os.path.join(reference, "src", "inquant")):
        return TARGET if os.path.isdir(os.path.join(TARGET, "inquant")) else None
    scratch = tempfile.mkdtemp(prefix="inquant_ref_")
    try:
        copy = os.path.join(scratch, "reference")
        shutil.copytree(reference, copy, ignore=shutil.ignore_patterns(".git", "docs", "benchmarks", "third_party"))
        if os.path.isdir(TARGET):
            shutil.rmtree(TARGET)
        for source in (copy, os.path.join(copy, "extensions", "vllm")):
            subprocess.run([sys.executable, "-m", "pip", "install", "--quiet", "--no-index", "--no-build-isolation", "--no-deps",
                            "--target", TARGET, source], check=True)
    finally:
        shutil.rmtree(scratch, ignore_errors=True)
    return TARGET


def available() -> bool:
    return os.path.isfile(os.path.join(TARGET, "inquant", "__init__.py"))


def load_reference(name: str = "inquant_reference"):
    """The reference's ``inquant`` package imported as ``name`` (its modules use relative imports).
    Transformers 5.x changed ``Cache.__init__``; with the import of transformers disabled the
    reference's cache falls back to its own stub base class, which is all the hot path needs."""
    if name in sys.modules:
        return sys.modules[name]
    if not available():
        raise ImportError("oracle/_ref is missing: run `python oracle/build_ref.py` where the reference checkout exists")
    path = os.path.join(TARGET, "inquant")
    spec = importlib.util.spec_from_file_location(name, os.path.join(path, "__init__.py"), submodule_search_locations=[path])
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    # a submodule that is already imported would be found without a look at its parent: hide both
    names = ("transformers", "transformers.cache_utils")
    hidden = {name: sys.modules.get(name, "absent") for name in names}
    for name in names:
        sys.modules[name] = None
    try:
        spec.loader.exec_module(module)
        for sub in ("codec", "value_codec", "cache"):
            importlib.import_module(f"{module.__name__}.{sub}")
    finally:
        for name, previous in hidden.items():
            if previous == "absent":
                sys.modules.pop(name, None)
            else:
                sys.modules[name] = previous
    return module


if __name__ == "__main__":
    print(build(*sys.argv[1:2]))
