"""CPU-side checks of the C-ABI boundary: the shared library builds, loads and
exports every function the header declares; the ctypes table mirrors the
header; the operators refuse to run without CUDA tensors (no CPU fallback)."""

import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "interattn_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ia_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib_path():
    from interattn_b200 import build
    return build.build()


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("ia_build_summaries", "ia_select", "ia_sparse_decode", "ia_finalize", "ia_workspace_bytes",
                 "ia_decode_attention", "ia_decode_attention_host", "ia_last_error_string", "ia_abi_version"):
        assert must in names


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(lib_path)
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_ctypes_table_matches_header(lib_path):
    from interattn_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_functions()
    lib = _lib.load()
    assert lib.ia_abi_version() == _lib.ABI_VERSION


def test_geometry_struct_layout_matches_the_header():
    from interattn_b200 import _lib
    assert ctypes.sizeof(_lib.Geom) == 12 * 4 + 2 * 8
    assert _lib.Geom.n_pool_pages.offset == 40
    assert _lib.Geom.pool_page_stride.offset == 48
    assert ctypes.sizeof(_lib.Summaries) == 7 * ctypes.sizeof(ctypes.c_void_p)  # k_bar k_max k_min v_bar v_norm_max w rho
    assert ctypes.sizeof(_lib.SelectAux) == 5 * ctypes.sizeof(ctypes.c_void_p)


def test_argument_validation_needs_no_gpu(lib_path):
    """Bad geometry is rejected before anything touches the device."""
    from interattn_b200 import _lib
    lib = _lib.load()
    g = _lib.Geom(batch=1, n_kv_heads=2, group_size=4, head_dim=96, page_size=16, block_size=64, max_pages=4,
                  max_blocks=1, dtype=_lib.IA_BF16, reserved=0, pool_page_stride=2 * 16 * 96, pool_head_stride=16 * 96)
    assert lib.ia_workspace_bytes(ctypes.byref(g), 4, 1, 0) == -1
    assert b"head_dim" in lib.ia_last_error_string()
    g.head_dim = 128
    g.pool_page_stride, g.pool_head_stride = 2 * 16 * 128, 16 * 128
    need = lib.ia_workspace_bytes(ctypes.byref(g), 4, 2, _lib.IA_REP_HYBRID)
    assert need > 0 and need % 256 == 0
    with pytest.raises(ValueError):
        _lib.check(lib.ia_finalize(None, None, 4, 1, 128, None, 0, None, None))
    # the pool size the block-table entries are checked against: never negative, spare field zero
    g.n_pool_pages = -3
    assert lib.ia_workspace_bytes(ctypes.byref(g), 4, 2, 0) == -1
    assert b"n_pool_pages" in lib.ia_last_error_string()
    g.n_pool_pages, g.reserved2 = 8, 1
    assert lib.ia_workspace_bytes(ctypes.byref(g), 4, 2, 0) == -1
    g.reserved2 = 0
    assert lib.ia_workspace_bytes(ctypes.byref(g), 4, 2, 0) > 0


def test_status_masks_match_the_header():
    from interattn_b200 import _lib
    text = open(HEADER).read()
    for name in ("SELECT_WAIT", "GEMM_WAIT", "PEER_WAIT", "BAD_INDEX"):
        m = re.search(rf"#define IA_DEV_STATUS_{name} (\d+)", text)
        assert m and int(m.group(1)) == getattr(_lib, f"IA_DEV_STATUS_{name}")


def test_operators_have_no_cpu_path():
    from interattn_b200 import ops
    q = torch.zeros(1, 8, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        ops.PagedKV(torch.zeros(4, 2, 16, 128), torch.zeros(4, 2, 16, 128), torch.zeros(1, 4, dtype=torch.int32),
                    torch.zeros(1, dtype=torch.int32), torch.zeros(1, dtype=torch.int32))
    with pytest.raises(ValueError, match="CUDA"):
        ops.finalize(torch.zeros(2, 1, 128), torch.zeros(2, 1), torch.float32)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from interattn_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _lib.load()
