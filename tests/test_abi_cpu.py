"""CPU-side checks of the C-ABI: the library builds for sm_100a, loads without a GPU and exports every symbol the header declares
(no compute call is made here)."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    with open(os.path.join(ROOT, "include", "wein_b200.h")) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(wein_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = _declared()
    for must in ("wein_b200_deltanet", "wein_b200_gdn_verify", "wein_b200_gdn_layer", "wein_b200_attn_verify", "wein_b200_paged_attn",
                 "wein_b200_gemm_wt", "wein_b200_accept_greedy", "wein_b200_accept_sampled", "wein_b200_topk_filter",
                 "wein_b200_engine_create", "wein_b200_engine_spec_step", "wein_b200_engine_spec_verify", "wein_b200_engine_draft",
                 "wein_b200_engine_warm", "wein_b200_engine_status", "wein_b200_gemm_wt_tc", "wein_b200_argmax_rows_noalloc"):
        assert must in names
    assert len(names) >= 40


def test_library_loads_and_exports_every_declared_symbol():
    from inferulm_b200 import build, lib
    build.build()
    so = lib.load()
    missing = [n for n in _declared() if not hasattr(so, n)]
    assert not missing, missing
    assert so.wein_b200_abi_version() == 2
    assert so.wein_b200_last_error() is not None


def test_library_exports_nothing_the_header_does_not_declare():
    """Every wein_b200_* symbol of the library is part of the declared C-ABI: no undeclared switches or hooks."""
    import subprocess
    from inferulm_b200 import build
    out = subprocess.run(["nm", "-D", "--defined-only", build.build()], capture_output=True, text=True, check=True).stdout
    exported = sorted({ln.split()[-1] for ln in out.splitlines() if ln.split() and ln.split()[-1].startswith("wein_b200_")})
    extra = [n for n in exported if n not in set(_declared())]
    assert not extra, extra


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from inferulm_b200 import lib
    monkeypatch.setattr(lib, "_lib", None)
    monkeypatch.setattr(lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(lib.LibraryMissing):
        lib.load()


def test_oracle_is_not_reachable_from_the_product():
    """The package never imports, includes or links the oracle (it is the checker, not a fallback)."""
    pkg = os.path.join(ROOT, "inferulm_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if not fn.endswith((".py", ".cu", ".cuh", ".h")):
                continue
            with open(os.path.join(dirpath, fn)) as f:
                src = f.read()
            assert not re.search(r"^\s*(from|import)\s+oracle\b", src, flags=re.M), fn
            assert "wein_oracle" not in src and "orc_" not in src and "libwein_oracle" not in src, fn
