"""CPU: the C-ABI library loads, exports every symbol include/b200moe.h declares, and refuses to
compute without a GPU (no fallback path)."""
import ctypes
import re
from ctypes import byref, c_void_p
from pathlib import Path

import pytest
import torch

from conftest import ROOT
from on_device_sd_b200 import _lib

HEADER = ROOT / "include" / "b200moe.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/b200moe.h but not exported"
    assert sorted(_lib.PROTOTYPES) == names, "python binding and header disagree on the symbol list"
    assert lib.b200moe_abi_version() == _lib.ABI_VERSION


def test_header_constants_match_binding():
    text = HEADER.read_text()
    for name, val in (("B200MOE_F32", _lib.F32), ("B200MOE_F16", _lib.F16), ("B200MOE_BF16", _lib.BF16),
                      ("B200MOE_W_DENSE", _lib.W_DENSE), ("B200MOE_W_INT4_G128", _lib.W_INT4_G128),
                      ("B200MOE_E_ARG", _lib.E_ARG), ("B200MOE_E_CUDA", _lib.E_CUDA), ("B200MOE_E_STATE", _lib.E_STATE),
                      ("B200MOE_MAX_EXPERTS", _lib.MAX_EXPERTS), ("B200MOE_MAX_TOPK", _lib.MAX_TOPK),
                      ("B200MOE_FFN_GEMV", _lib.FFN_GEMV), ("B200MOE_FFN_MMA", _lib.FFN_MMA)):
        m = re.search(rf"#define\s+{name}\s+(\d+)", text)
        assert m and int(m.group(1)) == val, name
    assert ctypes.sizeof(_lib.Config) == 40


def test_header_compiles_as_plain_c(tmp_path):
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    src = tmp_path / "t.c"
    src.write_text('#include "b200moe.h"\nint main(void){b200moe_config c; (void)c; return B200MOE_OK;}\n')
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-I", str(HEADER.parent), "-c", str(src), "-o", str(tmp_path / "t.o")], check=True)


def test_argument_errors_need_no_gpu():
    lib = _lib.load()
    h = c_void_p()
    assert lib.b200moe_create(None, byref(h)) == _lib.E_ARG
    bad = _lib.Config(32, 4, 5, 16, _lib.F16, _lib.W_DENSE, 1, 8, 0, 0)      # top_k > num_experts
    assert lib.b200moe_create(byref(bad), byref(h)) == _lib.E_ARG
    assert b"top_k" in lib.b200moe_last_error(None)
    bad = _lib.Config(36, 4, 2, 16, _lib.F16, _lib.W_DENSE, 1, 8, 0, 0)      # H not a multiple of 8
    assert lib.b200moe_create(byref(bad), byref(h)) == _lib.E_ARG
    bad = _lib.Config(32, 1000, 2, 16, _lib.F16, _lib.W_DENSE, 1, 8, 0, 0)   # too many experts
    assert lib.b200moe_create(byref(bad), byref(h)) == _lib.E_UNSUPPORTED
    bad = _lib.Config(128, 4, 2, 128, _lib.F16, _lib.W_INT4_G128, 1, 8, 0, 0)  # int4 needs bf16
    assert lib.b200moe_create(byref(bad), byref(h)) == _lib.E_UNSUPPORTED
    assert lib.b200moe_destroy(None) == _lib.OK
    assert lib.b200moe_pack_int4(None, 1, 128, _lib.BF16, None, None, None) == _lib.E_ARG
    assert lib.b200moe_route(None, 0, None, 1, None, None, None, None) == _lib.E_ARG


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU refusal")
def test_no_gpu_means_error_not_fallback():
    lib = _lib.load()
    h = c_void_p()
    ok = _lib.Config(32, 4, 2, 16, _lib.F16, _lib.W_DENSE, 1, 8, 0, 0)
    assert lib.b200moe_create(byref(ok), byref(h)) == _lib.E_CUDA
    assert b"no CPU path" in lib.b200moe_last_error(None)
    from on_device_sd_b200 import MoEContext
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        MoEContext(32, 4, 2, 16, torch.float16)


def test_product_package_never_touches_the_oracle():
    """The oracle is test infrastructure: no file of the package may import, read or name it."""
    pkg = ROOT / "on_device_sd_b200"
    for f in list(pkg.rglob("*.py")) + list(pkg.rglob("*.cu")) + list(pkg.rglob("*.cuh")):
        assert "oracle" not in f.read_text().lower(), f"{f} refers to the oracle"
