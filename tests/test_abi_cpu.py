"""CPU-side checks of the boundary: the C-ABI library loads and exports every symbol the public header
declares, and argument errors are reported before any device work (no compute call needs a GPU here)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def header_symbols():
    text = open(os.path.join(ROOT, "include", "ntb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ntb200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from neurotensor_b200 import _lib
    handle = _lib.lib()
    names = header_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(handle, n), "libntb200.so does not export %s" % n
    assert set(names) == set(_lib.SIGNATURES), "binding table and header disagree"


def test_header_is_plain_c(tmp_path):
    """The header compiles as C (no C++ or torch types in the signatures)."""
    import subprocess
    src = tmp_path / "t.c"
    src.write_text('#include "ntb200.h"\nint main(void){ntb200_gemm_desc d; (void)d; return 0;}\n')
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-c", str(src),
                           "-o", str(tmp_path / "t.o")])


def test_argument_errors_come_before_device_work():
    from neurotensor_b200 import _lib
    L = _lib.lib()
    # inner dimensions disagree -> invalid argument, with the reference's wording
    rc = L.ntb200_matmult(_lib.F32, None, None, None, 4, 5, 6, 7, 0, 0, None)
    assert rc == _lib.ERR_INVALID_ARG
    assert b"Expected second tensor rows to be 5 when it was 6" in L.ntb200_last_error_string()
    assert L.ntb200_matmult(99, None, None, None, 4, 5, 5, 7, 0, 0, None) == _lib.ERR_UNSUPPORTED
    # empty problems are a successful no-op
    assert L.ntb200_matmult(_lib.F32, None, None, None, 0, 5, 5, 7, 0, 0, None) == _lib.OK
    assert L.ntb200_gemm(None, None) == _lib.ERR_INVALID_ARG
    assert L.ntb200_conv2d(_lib.F16, None, None, None, None, 1, 3, 8, 8, 4, 3, 3, 0, 1, 0, 0, 1, 1,
                           None) == _lib.ERR_INVALID_ARG
    assert b"stride" in L.ntb200_last_error_string()


def test_no_device_is_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from neurotensor_b200 import _lib
    L = _lib.lib()
    n = ctypes.c_int(-1)
    rc = L.ntb200_device_count(ctypes.byref(n))
    assert rc in (_lib.ERR_NO_DEVICE, _lib.ERR_CUDA) or n.value == 0
    p = ctypes.c_void_p()
    assert L.ntb200_malloc_async(ctypes.byref(p), 1024, None) != _lib.OK


def test_python_mirror_rejects_cpu_tensors_and_bad_shapes():
    import torch
    from neurotensor_b200 import api
    a = torch.zeros(3, 4)
    with pytest.raises(ValueError):
        api.matmult(a, torch.zeros(4, 5))          # CPU tensors: there is no CPU path
    with pytest.raises(ValueError):
        api._matmult_shapes(a, torch.zeros(5, 5), False, False)
    with pytest.raises(ValueError):
        api._matmult_shapes(a, torch.zeros(4, 5, dtype=torch.float64), False, False)
    assert api._matmult_shapes(a, torch.zeros(3, 5), True, False)[:3] == (4, 3, 5)
    assert api._matmult_shapes(torch.zeros(2, 3, 4), torch.zeros(5, 4), False, True) == (3, 4, 5, (2,))
