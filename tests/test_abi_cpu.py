"""The C-ABI library loads without a GPU and exports every symbol include/nvfp4_b200.h declares;
host-side size helpers agree with the reference's formulas.  No compute calls here."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "nvfp4_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nvfp4_[a-z0-9_]+)\s*\(", text)))


def test_build_entry_compiles_and_imports():
    import __graft_entry__ as entry

    entry.build()
    assert os.path.exists(os.path.join(ROOT, "nanogpt-120a_b200", "libnvfp4_b200.so"))


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.library()
    declared = _declared_symbols()
    assert len(declared) >= 45
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(pkg.EXPORTED_SYMBOLS) == declared, "python binding and header disagree"
    assert lib.nvfp4_abi_version() == 3


def test_size_helpers(pkg):
    lib = pkg.library()
    # utils/nvfp4_tc_matmul/args.rs:37-39
    assert [lib.nvfp4_padded_k(k) for k in (1, 64, 65, 768, 8192)] == [64, 64, 128, 768, 8192]
    # utils/nvfp4_tma_matmul/scale_layout.rs: rows padded to 128, 512-byte tiles per (128 rows, 64 k)
    assert lib.nvfp4_scale_padded_mn_extent(129) == 256
    assert lib.nvfp4_scale_packed_len(8192, 768) == 8192 * 768 // 16
    assert lib.nvfp4_scale_packed_len(130, 128) == 2 * 2 * 512
    assert lib.nvfp4_tensor_amax_chunks(1025) == 2
    assert pkg.scale_packed_len(130, 128) == 2 * 2 * 512 and pkg.padded_k(65) == 128


def test_operations_fail_loudly_without_a_gpu(pkg):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError, match="CUDA device"):
        pkg.Nvfp4QuantModule().row_amax(torch.zeros(2, 16))
