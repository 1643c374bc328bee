"""pytest configuration: the `gpu` marker and import plumbing.

Tests marked `gpu` call the CUDA library through its C ABI and need a B200;
everything else runs on CPU.  The package directory name contains a hyphen, so
it is loaded by path under the module name `zkllm_ccs2024_b200`.
"""
import importlib.util
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def load_package():
    name = "zkllm_ccs2024_b200"
    if name in sys.modules:
        return sys.modules[name]
    pkg_dir = ROOT / "zkllm-ccs2024_b200"
    spec = importlib.util.spec_from_file_location(name, pkg_dir / "__init__.py",
                                                  submodule_search_locations=[str(pkg_dir)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def zkb():
    return load_package()


def pytest_sessionfinish(session, exitstatus):
    """With ZKLLM_GUARD=1 the library puts guard bands around every block it hands out (tests/test_gpu_guard.py); a
    session run that way fails if any band was written."""
    import ctypes
    import os
    z = sys.modules.get("zkllm_ccs2024_b200")
    if os.environ.get("ZKLLM_GUARD") != "1" or z is None:
        return
    blocks, damaged, first = ctypes.c_ulonglong(), ctypes.c_ulonglong(), ctypes.c_ulonglong()
    side = ctypes.c_int()
    try:
        z.call("zkb_guard_report", ctypes.byref(blocks), ctypes.byref(damaged), ctypes.byref(first), ctypes.byref(side), ctypes.c_int(0))
    except Exception:          # no device in this session
        return
    print(f"\n[guard] {blocks.value} blocks checked, {damaged.value} with a written guard band")
    if damaged.value:
        print(f"[guard] first: a block of {first.value} bytes, written {'before' if side.value == 0 else 'after'} it")
        session.exitstatus = 1
