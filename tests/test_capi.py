"""CPU checks of the C-ABI boundary: the library builds/loads and exports what the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
    text = open(os.path.join(ROOT, "include", "ghost_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ghost_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_expected_entry_points():
    names = _header_functions()
    for required in ("ghost_gram_dot_bf16", "ghost_wgrad_bf16", "ghost_persample_dot_bf16",
                     "ghost_colsum", "ghost_layernorm_persample", "ghost_embedding_dot",
                     "ghost_embedding_wgrad", "ghost_gradproj_dense_bf16", "ghost_last_error"):
        assert required in names


def test_library_builds_and_exports_every_declared_symbol():
    from ghostsuite_b200 import build, _lib
    path = build.build()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    for name in _header_functions():
        assert hasattr(lib, name), f"{name} declared in ghost_b200.h but not exported"
    # the ctypes prototypes cover exactly the header
    assert sorted(_lib.PROTOTYPES) == _header_functions()
    lib.ghost_version.restype = ctypes.c_char_p
    assert b"ghost_b200" in lib.ghost_version()


def test_ops_fail_loudly_without_cuda():
    import torch
    from ghostsuite_b200 import ops
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    A = torch.randn(4, 3, 8)
    with pytest.raises(RuntimeError):
        ops.gram_dot(A, A, 1)
    with pytest.raises(RuntimeError):
        ops.colsum(A)


def test_kernel_switches_validate_their_argument():
    """The process-wide kernel switches need no device: modes 0..2 are accepted, others rejected."""
    from ghostsuite_b200 import build
    lib = ctypes.CDLL(build.build())
    for name, default in (("ghost_set_persample_pair_mode", 1), ("ghost_set_wgrad_pair_mode", 1),
                          ("ghost_set_gram_pair_mode", 1)):
        fn = getattr(lib, name)
        fn.argtypes = [ctypes.c_int]
        fn.restype = ctypes.c_int
        assert fn(-1) < 0 and fn(3) < 0
        for mode in (0, 2, default):
            assert fn(mode) == 0
