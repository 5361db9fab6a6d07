"""The C-ABI library builds, loads, and exports every symbol its header declares.
No compute call is made here (no GPU needed)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "pr_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pr_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from retention_integration_b200 import build

    path = build.build()
    lib = ctypes.CDLL(path)
    names = _declared_symbols()
    assert len(names) >= 18
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/pr_b200.h but not exported"
    assert lib.pr_abi_version() == 1


def test_bad_arguments_return_codes_not_crashes():
    from retention_integration_b200 import _lib

    lib = _lib.lib()
    # null pointers / unsupported head dim are refused before any CUDA call
    rc = lib.pr_chunk_state(0, 1, 128, 1, 1, 32, 128, None, None, None, None, None, 1, 0, None)
    assert rc == -1 and b"head dim" in lib.pr_last_error()
    rc = lib.pr_discumsum_fwd(0, 1, 4, 4, 1, ctypes.c_longlong(7), None, None, None, None, None, 0, None)
    assert rc == -1
    rc = lib.pr_selftest_umma(9, 0, 64, 64, None, None, None, 0, None)
    assert rc == -1 and b"variant" in lib.pr_last_error()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from retention_integration_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    try:
        _lib.lib()
    except _lib.PRError as e:
        assert "no fallback" in str(e)
    else:
        raise AssertionError("a missing library must raise")


def test_cpu_tensors_are_rejected():
    import torch

    import retention_integration_b200 as prb

    q = torch.zeros(1, 128, 1, 64, dtype=torch.bfloat16)
    try:
        prb.power_retention(q, q, q, None, chunk_size=None)
    except prb.PRError as e:
        assert "CUDA" in str(e)
    else:
        raise AssertionError("CPU tensors must be rejected: there is no CPU path")
