"""The C-ABI library loads without a GPU and exports every function the headers declare."""
import ctypes as C
import os
import re

import pytest

import legion_ibp_b200 as L
from conftest import ROOT

DECL = re.compile(r"^\s*(?:const\s+)?(?:int|void|char)\s*\*?\s*(legion_\w+|BatchGenerate|RandomSample|"
                  r"FeatureCacheLookup|IOSubmit|IOComplete)\s*\(", re.M)


def declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(DECL.findall(text)))


def test_library_is_built_in_tree():
    assert os.path.exists(L.LIB_PATH), "run `make -C legion-ibp_b200/csrc` (or __graft_entry__.build())"
    assert os.path.dirname(L.LIB_PATH) == os.path.join(ROOT, "legion-ibp_b200")


@pytest.mark.parametrize("header", ["legion_b200.h", "legion_b200_compat.h"])
def test_every_declared_symbol_is_exported(header):
    lib = C.CDLL(L.LIB_PATH)
    names = declared(header)
    assert len(names) >= (5 if "compat" in header else 50), names
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_constants_and_layout_match_the_reference():
    lib = L.lib()
    assert lib.legion_abi_version() == 1
    lay = L.ipc_layout()
    # int32 steps[3] + cudaIpcMemHandle_t[8][2][7] of 64 bytes, no padding (ipc_service.cu:28-31)
    assert lay == dict(segment_bytes=12 + 8 * 2 * 7 * 64, handle_bytes=64, handles_offset=12)
    hdr = open(os.path.join(ROOT, "include", "legion_b200.h")).read()
    for name, val in (("LEGION_MAX_DEVICE", 8), ("LEGION_INTERBATCH_CON", 2), ("LEGION_INTRABATCH_CON", 3),
                      ("LEGION_MEMORY_USAGE", 7), ("LEGION_CACHEMISS_FLAG", "(-2)"), ("LEGION_MAX_FANOUT", 32)):
        assert re.search(r"#define %s\s+%s(?!\w)" % (name, re.escape(str(val))), hdr), name


def test_argument_errors_do_not_need_a_gpu():
    lib = L.lib()
    h = C.c_void_p()
    assert lib.legion_graph_create(C.byref(h), 0, C.c_int64(0), C.c_int64(0), None, None) == -1
    assert b"NULL" in lib.legion_last_error() or b"n_nodes" in lib.legion_last_error()
    assert lib.legion_ipc_create(C.byref(h), 9, None) == -1
    assert lib.legion_pool_set_rng(None, C.c_uint64(1), 64) == -1
    assert lib.legion_copy(None, None, C.c_int64(8), 1) == -1


def test_python_mirror_fails_loudly_without_the_library(monkeypatch, tmp_path):
    monkeypatch.setattr(L, "LIB_PATH", str(tmp_path / "nope.so"))
    monkeypatch.setattr(L, "_lib", None)
    with pytest.raises(L.LegionError, match="no CPU fallback"):
        L.lib()
