"""The ahead-of-time build when several processes (the ranks of one job) find the library stale at once."""
import os
import subprocess
import sys

from autogptq.tvm_b200 import build as B

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_concurrent_imports_build_once_and_all_load():
    """Three processes call build() while the library is older than its sources: the file lock lets one of them build,
    the others wait and find it fresh; every one of them then loads a complete library (all symbols bind)."""
    assert os.path.isfile(B.LIB_PATH)
    os.utime(B.LIB_PATH, (1, 1))          # older than every source: stale
    assert B.is_stale()
    code = ("import sys; sys.path.insert(0, %r); "
            "from autogptq.tvm_b200 import build as B; B.build(); "
            "from autogptq.tvm_b200 import _lib; print(len(_lib._SIGNATURES))") % REPO
    procs = [subprocess.Popen([sys.executable, "-c", code], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
             for _ in range(3)]
    outs = [p.communicate(timeout=600) for p in procs]
    for p, (out, err) in zip(procs, outs):
        assert p.returncode == 0, err[-2000:]
        assert int(out.strip().splitlines()[-1]) > 20
    assert not B.is_stale()
    leftovers = [f for f in os.listdir(os.path.dirname(B.LIB_PATH)) if ".so.tmp" in f]
    assert not leftovers
