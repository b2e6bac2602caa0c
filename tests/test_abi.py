"""The C-ABI library loads without a GPU and exports every function include/mlc_b200.h
declares; the host-only parts of it work; device entry points fail loudly, never fall back."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_functions():
    text = (ROOT / "include" / "mlc_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(mlc_[a-z0-9_]+)\s*\(", text))
    # function-pointer typedefs and struct members are not exports
    names -= set(re.findall(r"\(\*\s*(mlc_[a-z0-9_]+)\s*\)", text))
    return sorted(names)


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ("mlc_run_paged_flash_attention", "mlc_encode_paged_flash_attention",
                 "mlc_run_scatter_kv_paged_batched_f16", "mlc_encode_scatter_kv_paged_batched_f16",
                 "mlc_run_scatter_kv_paged", "mlc_run_gather_kv_pages", "mlc_pass_begin", "mlc_pass_flush",
                 "mlc_alloc", "mlc_cached_buffer", "mlc_page_pool_create", "mlc_scheduler_create"):
        assert must in names
    assert len(names) >= 80


def test_library_exports_every_declared_symbol(lib):
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_no_device_means_an_error_not_a_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("this check is for machines without a GPU")
    import mlcompiler_b200
    with pytest.raises(mlcompiler_b200.MlcError) as e:
        mlcompiler_b200.Executor(0)
    assert e.value.status == 6   # MLC_ERR_NO_DEVICE


def test_product_package_does_not_touch_the_oracle():
    """The oracle is test infrastructure: nothing under mlcompiler_b200/ may import or load it."""
    for path in (ROOT / "mlcompiler_b200").rglob("*"):
        if path.suffix in (".py", ".cu", ".cpp", ".hpp", ".h") and path.is_file():
            text = path.read_text()
            assert "import oracle" not in text and "from oracle" not in text, path
            assert "paged_oracle" not in text and "libref_attention" not in text, path


def test_missing_library_is_a_loud_import_error(monkeypatch, tmp_path):
    import mlcompiler_b200.capi as capi
    monkeypatch.setattr(capi, "_LIB", None)
    monkeypatch.setattr(capi, "_PKG", tmp_path)
    with pytest.raises(ImportError):
        capi.load_library()


def test_exchange_layout_keeps_every_slot_16_byte_aligned():
    """Gather-buffer layout of the peer exchange (pure host arithmetic): with head_dim % 4 == 0 a
    slot of max_rows * (head_dim + 2) floats is only a multiple of 4 floats when max_rows is even;
    the layout rounds it up, so that the float4 stores and loads of the kernel stay aligned for an
    odd max_rows, on every (parity, rank) slot, and the flag words follow behind the last slot."""
    import ctypes as C
    import mlcompiler_b200
    lib = mlcompiler_b200.load_library(build_if_missing=True)
    for world in (1, 2, 3, 8, 16):
        for max_rows in (1, 3, 127, 128, 129, 4097):
            for D in (4, 64, 128):
                slot, flags, total = C.c_size_t(), C.c_size_t(), C.c_size_t()
                assert lib.mlc_exchange_layout(world, max_rows, D, C.byref(slot), C.byref(flags), C.byref(total)) == 0
                assert slot.value % 4 == 0 and slot.value >= max_rows * (D + 2)
                for parity in (0, 1):
                    for rank in range(world):
                        assert ((parity * world + rank) * slot.value * 4) % 16 == 0
                assert flags.value % 256 == 0 and flags.value >= 2 * world * slot.value * 4
                assert total.value >= flags.value + 2 * world * 4 + 8
    assert lib.mlc_exchange_layout(0, 8, 64, None, None, None) != 0
    assert lib.mlc_exchange_layout(2, 8, 66, None, None, None) != 0
