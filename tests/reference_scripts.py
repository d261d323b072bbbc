"""Finding and importing the reference's own Python side (scripts/jiuge.py, scripts/infer_task.py,
scripts/kvcache_pool.py, scripts/libinfinicore_infer.py) for the tests that hold this package against it.

The reference's binding opens ``$INFINI_ROOT/lib/libinfinicore_infer.so`` when it is imported
(scripts/libinfinicore_infer.py:84-88).  Its model code cannot be built here (it calls the external InfiniCore
libraries), but the Python classes that read a configuration, pack the weights and marshal a batch run on the CPU
given ANY shared object that exports the six symbols; ``stub_library`` compiles one whose functions do nothing.
"""
import importlib
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_STUB = """
void *createJiugeModel(void) { return 0; }
void destroyJiugeModel(void) {}
void *createKVCache(void) { return 0; }
void dropKVCache(void) {}
void inferBatch(void) {}
void forwardBatch(void) {}
"""


def scripts_dir():
    """The folder of the reference's scripts, or None: ``$INFINICORE_INFER_REFERENCE``, the reference installed
    beside the benchmark (``baseline/_ref``), or a checkout next to this repository."""
    for base in (os.environ.get("INFINICORE_INFER_REFERENCE"), os.path.join(ROOT, "baseline", "_ref"),
                 os.path.join(os.path.dirname(ROOT), "reference")):
        if base and os.path.isfile(os.path.join(base, "scripts", "jiuge.py")):
            return os.path.join(base, "scripts")
    return None


def stub_library(folder: str) -> str:
    """``folder/lib/libinfinicore_infer.so`` with the six symbols, doing nothing; returns ``folder``."""
    os.makedirs(os.path.join(folder, "lib"), exist_ok=True)
    src = os.path.join(folder, "stub.c")
    with open(src, "w") as f:
        f.write(_STUB)
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        raise RuntimeError("no C compiler")
    subprocess.run([cc, "-shared", "-fPIC", "-o", os.path.join(folder, "lib", "libinfinicore_infer.so"), src], check=True)
    return folder


def import_reference(infini_root: str, names=("jiuge",)):
    """Import the reference's modules by their own top-level names with ``INFINI_ROOT`` pointing at a library."""
    d = scripts_dir()
    if d is None:
        raise ImportError("the reference's scripts are not on this machine")
    os.environ["INFINI_ROOT"] = infini_root
    if d not in sys.path:
        sys.path.insert(0, d)
    return [importlib.import_module(n) for n in names]
