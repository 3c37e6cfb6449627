"""The allocation-free embedding entry point against the workspace-taking one.

Some callers may not allocate device memory when the hook fires (their memory belongs to a fixed
pool, or they run inside a section where re-entering an allocator would deadlock), so they cannot
give ghost_embedding_dot a workspace.  ghost_embedding_dot_noalloc keeps its tables in a device
array inside the library instead.  This file is collected last on purpose: if it fails, a run that
stops at the first failure has already run everything else.
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
