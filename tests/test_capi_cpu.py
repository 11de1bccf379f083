"""CPU checks of the C ABI: the library loads, exports every symbol the headers
declare, and rejects bad arguments with a status (no compute without a GPU)."""
import ctypes
import os
import re

import pytest

import __graft_entry__ as ge

ROOT = ge.ROOT


@pytest.fixture(scope="module")
def library():
    ge.build()
    return ge.load_package().lib()


def declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(polar_b200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(library):
    names = declared("polar_b200.h")
    assert len(names) >= 20
    for name in names:
        assert hasattr(library.cdll, name), name


def test_binding_table_matches_header(library):
    from polarai_framework_b200.capi import SIGNATURES
    assert sorted(SIGNATURES) == declared("polar_b200.h")


def test_bad_arguments_return_status_not_abort(library):
    c = library.cdll
    assert c.polar_b200_ffill(1.0, None, 4, None) == 1
    assert "null" in library.last_error()
    assert c.polar_b200_fadd(None, 1.0, None, 1.0, None, 0, None) == 0      # n == 0 is a no-op
    assert c.polar_b200_fmatmul(2, 0, 4, 4, 4, None, None, None, None, 0, None) == 1
    assert c.polar_b200_fmatmul(0, 0, 0, 4, 4, None, None, None, None, 0, None) == 0
    assert c.polar_b200_launch_by_name(b"fnope", None, 0, None, 0, None) == 3
    assert c.polar_b200_launch_by_name(None, None, 0, None, 0, None) == 1
    assert library.launch_count() == 0


def test_launch_by_name_checks_argument_patterns(library):
    from polarai_framework_b200.capi import Arg
    c = library.cdll
    shape = (ctypes.c_uint64 * 1)(4)
    args = (Arg * 2)()
    for a in args:
        a.is_tensor = 1
        a.tensor.dims = 1
        a.tensor.shape = shape
    assert c.polar_b200_launch_by_name(b"fadd", args, 2, None, 0, None) == 3   # wrong arity
    assert c.polar_b200_launch_by_name(b"fmatmul_f_f", args, 2, None, 0, None) == 3


def test_matmul_path_selection(library):
    c = library.cdll
    assert c.polar_b200_fmatmul_path(0, 0, 8192, 8192, 8192) == 0     # tensor cores
    assert c.polar_b200_fmatmul_path(0, 0, 65536, 4096, 784) == 0
    assert c.polar_b200_fmatmul_path(1, 0, 784, 4096, 65536) == 0
    assert c.polar_b200_fmatmul_path(0, 0, 65536, 10, 4096) != 0      # row pitch 40 B: no TMA
    assert c.polar_b200_fmatmul_path(0, 0, 256, 1, 784) != 0


def test_runtime_plugin_exports_and_opens_without_a_gpu(library):
    from polarai_framework_b200 import runtime
    cdll = runtime.load_rt_library()           # resolves every declared symbol + initContext/closeContext
    assert sorted(runtime.RT_SIGNATURES) == declared("polar_b200_rt.h")
    import torch
    if not torch.cuda.is_available():
        rt = runtime.Runtime()
        assert rt.device_count() == 0          # no sm_100 device: an empty context, not a crash
        with pytest.raises(Exception):
            rt.tensor((4,))
        rt.close()
