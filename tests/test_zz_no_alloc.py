"""The allocation-free embedding entry point against the workspace-taking one.

Some callers may not allocate device memory when the hook fires (their memory belongs to a fixed
pool, or they run inside a section where re-entering an allocator would deadlock), so they cannot
give ghost_embedding_dot a workspace.  ghost_embedding_dot_noalloc keeps its tables in a device
array inside the library instead.  The file name sorts last so that this add-on entry point is
exercised after the entry points every engine depends on: a run stopped at its first failure
(`pytest -x`) has then already covered those, and the shared array is also met in whatever state
the rest of the session left the device in.
"""
import ctypes

import pytest
import torch

from oracle import ghost_oracle as O

pytestmark = pytest.mark.gpu


def _call_both(lib, ids, G, n_train, n_val, vocab):
    from ghostsuite_b200 import _lib
    N, T, d = G.shape
    stream = torch.cuda.current_stream().cuda_stream
    is_f32 = 1 if G.dtype == torch.float32 else 0
    M_ws = torch.full((n_val, n_train), float("nan"), device="cuda")
    ws_bytes = int(lib.ghost_embedding_dot_workspace_bytes(n_val, T, vocab))
    ws = torch.empty(ws_bytes + 256, dtype=torch.uint8, device="cuda")
    _lib.check(lib.ghost_embedding_dot(ids.data_ptr(), G.data_ptr(), is_f32, n_train, n_val, T, d, vocab,
                                       1.0, M_ws.data_ptr(), ws.data_ptr(), ws_bytes, stream))
    M_na = torch.full((n_val, n_train), float("nan"), device="cuda")
    _lib.check(lib.ghost_embedding_dot_noalloc(ids.data_ptr(), G.data_ptr(), is_f32, n_train, n_val, T, d,
                                               vocab, 1.0, M_na.data_ptr(), stream))
    torch.cuda.synchronize()
    return M_ws, M_na


def test_noalloc_entry_point_matches_workspace_entry_point_twice_in_a_row():
    from ghostsuite_b200 import _lib
    lib = _lib.load()
    g = torch.Generator().manual_seed(12)
    # two different problems back to back: the second call finds the first call's tables in the
    # shared array and must not be affected by them
    for (n_train, n_val, T, d, vocab, dtype) in ((6, 3, 50, 64, 97, torch.bfloat16),
                                                 (4, 2, 33, 24, 1000, torch.float32)):
        N = n_train + n_val
        ids = torch.randint(0, vocab, (N, T), generator=g).cuda()
        G = (torch.randn(N, T, d, generator=g) / d ** 0.5).to(dtype).cuda()
        M_ws, M_na = _call_both(lib, ids, G, n_train, n_val, vocab)
        ref = O.embedding_dot_exact(ids.cpu(), G.cpu(), n_val)
        tol = 1e-5 if dtype == torch.float32 else 1e-4      # same tolerances as test_kernels_gpu.py
        assert O.rel_fro(M_na, M_ws) < tol
        assert O.rel_fro(M_na, ref) < tol
    _lib.poll_kernel_error()


def test_noalloc_entry_point_rejects_sizes_beyond_its_scratch():
    from ghostsuite_b200 import _lib
    lib = _lib.load()
    ids = torch.zeros((3, 4), dtype=torch.int64, device="cuda")
    G = torch.zeros((3, 4, 8), device="cuda")
    M = torch.zeros((1, 2), device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.ghost_embedding_dot_noalloc(ids.data_ptr(), G.data_ptr(), 1, 2, 1, 4, 8, 131073, 1.0,
                                         M.data_ptr(), stream)
    assert rc == _lib.GHOST_ERR_INVALID and b"exceeds the built-in scratch" in lib.ghost_last_error()
    rc = lib.ghost_embedding_dot_noalloc(ids.data_ptr(), G.data_ptr(), 1, 2, 1, 131073, 8, 100, 1.0,
                                         M.data_ptr(), stream)
    assert rc == _lib.GHOST_ERR_INVALID and b"exceeds the built-in scratch" in lib.ghost_last_error()


def test_noalloc_entry_point_allocates_nothing_and_fills_its_scratch_exactly():
    """The property the entry point exists for: once its first call on the device has looked up the
    array's address, a call takes no device memory at all (free memory as the driver reports it is
    unchanged across the call).  The problem is the largest the 1 MiB array holds -- vocab = 131072
    head entries and n_val * T = 131072 chain entries -- and is checked against the workspace entry
    point."""
    from ghostsuite_b200 import _lib
    lib = _lib.load()
    n_train, n_val, T, d, vocab = 3, 2, 65536, 8, 131072
    g = torch.Generator().manual_seed(13)
    ids = torch.randint(0, vocab, (n_train + n_val, T), generator=g).cuda()
    ids[n_train, 0] = vocab - 1                                   # the last head entry is used
    ids[0, 5] = vocab - 1
    G = torch.randn(n_train + n_val, T, d, generator=g).cuda()
    M_ws, M_na = _call_both(lib, ids, G, n_train, n_val, vocab)   # also the warm-up call of this device
    assert O.rel_fro(M_na, M_ws) < 1e-5
    stream = torch.cuda.current_stream().cuda_stream
    M2 = torch.full((n_val, n_train), float("nan"), device="cuda")
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    _lib.check(lib.ghost_embedding_dot_noalloc(ids.data_ptr(), G.data_ptr(), 1, n_train, n_val, T, d, vocab,
                                               1.0, M2.data_ptr(), stream))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before and torch.cuda.memory_reserved() == reserved_before
    assert O.rel_fro(M2, M_ws) < 1e-5
    _lib.poll_kernel_error()
