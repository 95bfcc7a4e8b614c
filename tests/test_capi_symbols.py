"""The C-ABI library loads and exports every symbol include/ra_spmm_b200.h declares."""
import ctypes as C
import re
from pathlib import Path

from ra_spmm_b200 import _capi

HEADER = Path(__file__).resolve().parent.parent / "include" / "ra_spmm_b200.h"


def declared_symbols():
    text = HEADER.read_text()
    return re.findall(r"RA_API\s+[\w\s\*]+?\b(ra_\w+)\s*\(", text)


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert set(names) == set(_capi.EXPORTED_SYMBOLS)


def test_host_only_entry_points(lib):
    assert lib.ra_version() >= 100
    assert lib.ra_path_name(13) == b"ZERO_OVERHEAD_CSR"
    assert lib.ra_path_name(99) == b"UNKNOWN"
    # argument errors are reported through the status code and the error string
    assert lib.ra_route(None, 0, None) == 1
    assert b"null" in lib.ra_last_error_string()
    assert lib.ra_zo_plan_info(None, None) == 1
    assert lib.ra_tile_plan_destroy(None) == 0


def test_struct_sizes_match_header():
    # layout the C compiler gives the header's structs (x86-64 SysV)
    assert C.sizeof(_capi.RaFeatures) == 48
    assert C.sizeof(_capi.RaRoute) == 92


def test_fnv1a64_known_vectors(lib):
    import ctypes
    for text, want in ((b"", 0xcbf29ce484222325), (b"a", 0xaf63dc4c8601ec8c), (b"foobar", 0x85944171f73967e8)):
        buf = ctypes.create_string_buffer(text, len(text)) if text else None
        assert lib.ra_fnv1a64_host(buf, len(text)) == want


def test_plan_checksum_hook_prints_fnv1a_per_array(monkeypatch, capsys):
    """RA_PLAN_CHECKSUM=1 makes the plan constructors report FNV-1a checksums on stderr
    (the hook experiments/verify_format_checksums.py relies on). Checked here on a stand-in
    plan object; the constructors call the same function on real plans."""
    import numpy as np
    import torch
    from ra_spmm_b200 import ra_spmm
    from ra_spmm_b200.harness import fnv1a64

    class FakePlan:
        def arrays(self):
            return {"a": torch.tensor([1, 2, 3], dtype=torch.int32), "none": torch.empty(0, dtype=torch.int32)}

    monkeypatch.delenv("RA_PLAN_CHECKSUM", raising=False)
    ra_spmm._report_checksum("FakePlan", FakePlan())
    assert capsys.readouterr().err == ""
    monkeypatch.setenv("RA_PLAN_CHECKSUM", "1")
    ra_spmm._report_checksum("FakePlan", FakePlan())
    err = capsys.readouterr().err
    want = fnv1a64(np.array([1, 2, 3], dtype=np.int32))
    assert err.startswith("[RA_PLAN_CHECKSUM] FakePlan ")
    assert f"a={want:016x}" in err and "none=cbf29ce484222325" in err and " all=" in err


def test_plan_file_errors_come_before_any_device_work(lib, tmp_path):
    """Header checks of the plan-file readers (no GPU needed: they fail before the first allocation)."""
    out = C.c_void_p()
    assert lib.ra_tile_plan_load(str(tmp_path / "missing.plan").encode(), C.byref(out)) == 1
    assert b"cannot open" in lib.ra_last_error_string() and not out.value
    bad = tmp_path / "bad.plan"
    bad.write_bytes(b"NOTAPLAN" + bytes(200))
    assert lib.ra_zo_plan_load(str(bad).encode(), C.byref(out)) == 1
    assert b"bad magic" in lib.ra_last_error_string()
    bad.write_bytes(b"RASPMMB2" + (7).to_bytes(4, "little") + bytes(200))
    assert lib.ra_zo_plan_load(str(bad).encode(), C.byref(out)) == 3          # RA_ERR_UNSUPPORTED: version
    bad.write_bytes(b"RASPMMB2" + (1).to_bytes(4, "little") + (1).to_bytes(4, "little") + bytes(16 * 8))
    assert lib.ra_zo_plan_load(str(bad).encode(), C.byref(out)) == 1          # a tile file given to the ZERO_OVERHEAD reader
    assert b"tile" in lib.ra_last_error_string()
    assert lib.ra_zo_plan_save(None, b"x") == 1
