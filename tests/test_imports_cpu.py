"""Every module of the package imports on a machine without a GPU (syntax errors and missing names in modules that
only GPU runs exercise show up here), and the entry points parse their own ``--help``."""
import importlib
import os
import pkgutil
import subprocess
import sys

import distca_b200

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_module_imports():
    names = [m.name for m in pkgutil.walk_packages(distca_b200.__path__, prefix="distca_b200.")]
    assert len(names) > 30
    for name in names:
        if name.rsplit(".", 1)[-1] in ("_planner", "_kernels"):      # the native libraries (one is loaded with ctypes)
            continue
        importlib.import_module(name)
    for name in distca_b200.__all__:
        assert getattr(distca_b200, name) is not None


def test_entry_points_print_their_help():
    for script in ("bench.py", "pretrain_llama.py"):
        r = subprocess.run([sys.executable, os.path.join(ROOT, script), "--help"], capture_output=True, text=True, timeout=120)
        assert r.returncode == 0 and "usage:" in r.stdout, r.stderr[-1000:]
    for mod in ("distca_b200.sweep", "distca_b200.launch", "distca_b200.utils.net_bench", "distca_b200.utils.kernel_bench",
                "distca_b200.utils.fa2a_bench", "distca_b200.runtime.selfcheck", "distca_b200.planner.tools",
                "distca_b200.utils.guards"):
        r = subprocess.run([sys.executable, "-m", mod, "--help"], capture_output=True, text=True, timeout=120, cwd=ROOT)
        assert r.returncode == 0 and "usage:" in r.stdout, (mod, r.stderr[-1000:])
