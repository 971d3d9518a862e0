"""The C-ABI library loads without a GPU and exports every symbol include/pat_b200.h declares;
host-only entry points behave; device entry points refuse to run without a device."""
import ctypes as C
import os
import re

import pytest

from pat_b200 import _native as N

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "pat_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pat_(?:b200|tree|work)_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(native_lib):
    names = _declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(native_lib, name), f"{name} is declared but not exported"
        assert name in N.SIGNATURES, f"{name} is exported but has no ctypes signature"
    assert sorted(N.SIGNATURES) == names


def test_structs_match_the_header_sizes(native_lib):
    # pat_work_header: 18 int32 + 5 int64 + 4 int32; pat_work_options: 10 int32; pat_plan_bucket: 4 int32 + 4 ptr
    assert C.sizeof(N.WorkHeader) == 18 * 4 + 5 * 8 + 4 * 4
    assert C.sizeof(N.WorkOptions) == 40
    assert C.sizeof(N.PlanBucket) == 16 + 4 * 8
    assert C.sizeof(N.BucketView) == 24 + 5 * 8


def test_version_and_strerror(native_lib):
    assert native_lib.pat_b200_abi_version() >= 4
    assert N.strerror(0) == "ok"
    assert "workspace" in N.strerror(-12)
    assert N.strerror(-999) == "unknown status"


def test_tree_handle_lifecycle_and_errors(native_lib):
    assert native_lib.pat_tree_create(0, 0) is None
    assert native_lib.pat_tree_create(16, 7) is None
    t = native_lib.pat_tree_create(16, N_SEM := 1)
    assert t
    assert native_lib.pat_tree_pack(t, None, 0, 4, 8, 0) == -5          # not built yet
    lens = (C.c_int32 * 2)(20, 40)
    table = (C.c_int32 * 6)(1, 2, 0, 1, 3, 4)
    assert native_lib.pat_tree_build(t, lens, table, 2, 3) == 0
    assert native_lib.pat_tree_build(t, lens, table, 2, 3) == -1         # one build per tree
    assert native_lib.pat_tree_pack(t, None, 0, 0, 8, 0) == -1           # HRatio must be positive
    assert native_lib.pat_tree_pack(t, None, 0, 4, 8, 0) == 0
    assert native_lib.pat_tree_num_buckets(t) >= 1
    mx = (C.c_int32 * 3)()
    assert native_lib.pat_tree_maxima(t, mx) == 0 and mx[0] >= 1
    native_lib.pat_tree_destroy(t)
    native_lib.pat_tree_destroy(None)


def test_decode_rejects_bad_arguments_without_touching_a_device(native_lib):
    assert native_lib.pat_b200_decode(None, None) == -1
    a = N.DecodeArgs()
    assert native_lib.pat_b200_decode(C.byref(a), None) == -1
    hdr = N.WorkHeader()
    hdr.num_entries = 10            # 10 slots of hratio rows each
    hdr.hratio = 4
    assert native_lib.pat_b200_workspace_bytes(C.byref(hdr), 8, 128) >= 10 * 4 * 129 * 4
    assert native_lib.pat_b200_workspace_bytes(None, 8, 128) == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(N, "_lib", None)
    monkeypatch.setattr(N, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        N.load()
