"""CPU: the C-ABI library loads and exports every function include/zkllm_b200.h
declares; host-only behaviour (no kernel launches)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol(zkb):
    lib = zkb.lib()
    declared = zkb.exported_symbols_from_header()
    assert len(declared) > 60
    missing = [s for s in declared if not hasattr(lib, s)]
    assert missing == []


def test_header_cites_the_reference_for_every_entry_point():
    """each entry point is documented with the reference file:line it replaces, or
    says that it has no counterpart"""
    text = (ROOT / "include" / "zkllm_b200.h").read_text()
    blocks = re.split(r"\n(?=/\*)", text)
    cited = 0
    for b in blocks:
        if "zkb_" in b and ("int zkb_" in b or "long zkb_" in b or "char* zkb_" in b):
            assert re.search(r"\.cuh?:\d+|no counterpart|ctors, dtors|library", b), b[:200]
            cited += 1
    assert cited >= 20


def test_version_error_text_and_launch_counter(zkb):
    lib = zkb.lib()
    assert lib.zkb_version() >= 100
    assert isinstance(lib.zkb_last_error(), bytes)
    assert zkb.launch_count() >= 0


def test_missing_library_fails_loudly(zkb, monkeypatch, tmp_path):
    monkeypatch.setattr(zkb, "_lib", None)
    monkeypatch.setattr(zkb, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(FileNotFoundError):
        zkb.lib()


def test_product_sources_do_not_touch_the_oracle():
    """the library and its Python binding never import, include or link oracle/"""
    pkg = ROOT / "zkllm-ccs2024_b200"
    for p in list(pkg.rglob("*.cu")) + list(pkg.rglob("*.cuh")) + list(pkg.rglob("*.hpp")) + list(pkg.rglob("*.py")):
        txt = p.read_text()
        assert "oracle" not in txt and "pyref" not in txt, p
