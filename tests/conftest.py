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
