"""The C-ABI library loads and exports every symbol the public header declares (no compute)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "odmkv_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(odmkv_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_expected_groups():
    syms = header_symbols()
    for s in ("odmkv_score_prefill", "odmkv_allocate_bits", "odmkv_quantize_pack", "odmkv_dequant_chunk",
              "odmkv_decode_attn", "odmkv_export_bank"):
        assert s in syms


def test_library_exports_every_declared_symbol(pkg):
    pkg.build.build_library()
    handle = ctypes.CDLL(pkg._lib.LIB_PATH)
    missing = [s for s in header_symbols() if not hasattr(handle, s)]
    assert not missing, missing
    assert handle.odmkv_abi_version() == 1


def test_binding_covers_header(pkg):
    bound = set(pkg._lib._PROTOTYPES) | set(pkg._lib._OPTIONAL)
    assert set(header_symbols()) <= bound


def test_struct_sizes_match(pkg):
    # odmkv_chunk: 24 pointers + 6 + 4 int32; report: 2 doubles + 8 int64 + 6 int32
    assert ctypes.sizeof(pkg._lib.Chunk) == 26 * 8 + 10 * 4
    assert ctypes.sizeof(pkg._lib.AllocReport) == 16 + 64 + 24


def test_status_strings_and_host_queries(pkg):
    L = pkg._lib.lib()
    assert L.odmkv_status_string(0) == b"ok"
    assert b"shape" in L.odmkv_status_string(-2)
    assert L.odmkv_pack_plan_workspace_bytes(1, 8, 4096) == 2 * 8 * 32 * 6 * 4
    assert L.odmkv_alloc_num_rounds(6) == 74 + 25
    assert L.odmkv_alloc_num_rounds(1) == 1
    assert L.odmkv_decode_default_splits(1, 8, 131072) == 38 and L.odmkv_decode_default_splits(8, 8, 131072) == 6
    assert L.odmkv_score_workspace_bytes(1, 8, 4, 4096) > 8 * 4 * 4096 * 4
