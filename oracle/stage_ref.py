"""Stage the reference's own CPU implementation of the path for use as a checker / timed baseline.

The reference's torch dequantise-then-matmul path is one self-contained Python file
(``auto_gptq/nn_modules/qlinear.py`` of LeiWang1999/AutoGPTQ.tvm, forward at lines 197-243).  This recipe
copies that file, unmodified, from a reference checkout into ``oracle/_ref/`` (a directory that is kept out of
version control) so that it can be loaded by path where the checkout itself is not available.  Nothing here is
part of the product, and the product never imports ``oracle/``.

    python oracle/stage_ref.py [/path/to/reference]      (default: $B200GPTQ_REFERENCE)
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
REF_FILE = os.path.join(REF_DIR, "qlinear.py")
REL = os.path.join("auto_gptq", "nn_modules", "qlinear.py")


def stage(reference_root=None) -> str:
    """Copy the file if a checkout is given / configured; return the staged path or "" when there is none."""
    root = reference_root or os.environ.get("B200GPTQ_REFERENCE", "")
    src = os.path.join(root, REL) if root else ""
    if src and os.path.isfile(src):
        os.makedirs(REF_DIR, exist_ok=True)
        shutil.copyfile(src, REF_FILE)
    return REF_FILE if os.path.isfile(REF_FILE) else ""


def load():
    """The staged reference module (loaded by path, its prints silenced by the caller), or None."""
    if not os.path.isfile(REF_FILE):
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("b200gptq_reference_qlinear", REF_FILE)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    path = stage(sys.argv[1] if len(sys.argv) > 1 else None)
    print(path or "no reference checkout given: nothing staged")
