"""The allocation-free routing-count entry point, called through its exported C symbol.

Some callers cannot allocate device memory where they need the counts (a host program without
PyTorch, code running under a memory pool that forbids raw allocation, a region that must not
synchronise the device).  For them the library exports one C function that takes caller-owned
input and output buffers and keeps its intermediate histograms in a fixed array inside the library.
This test calls that symbol with ctypes, twice in a row on different inputs (the second smaller,
so leftovers of the first call would show), and compares with the counts of the regular path and
with an independent count made by torch.bincount.  It is collected last on purpose.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular_counts(idx, E, N):
    import teramoe_b200 as tm
    from teramoe_b200._build import load_ext

    ext = load_ext()
    T, K = idx.shape
    C = E + N + 2
    chunk = ext.route_chunk_tokens()
    chunks = max(1, (T + chunk - 1) // chunk)
    hist = torch.zeros(chunks * C, dtype=torch.int32, device=idx.device)
    ext.route_hist(idx, E, N, hist)
    return hist.view(chunks, C).sum(0, dtype=torch.int32)


def _bincount_counts(idx, E, N):
    """The same counts from library ops only (no kernel of this repository)."""
    T, K = idx.shape
    i = idx.long()
    valid = (i >= 0) & (i < E)
    per_expert = torch.bincount(i[valid], minlength=E)
    dst = torch.where(valid, i // (E // N), torch.full_like(i, N))
    hit = torch.zeros(T, N + 1, dtype=torch.long, device=idx.device).scatter_(1, dst, 1)[:, :N]
    return torch.cat([per_expert, hit.sum(0), hit.sum().view(1), torch.tensor([T], device=idx.device)]).to(torch.int32)


def test_no_alloc_route_counts_two_calls():
    from teramoe_b200 import _build

    _build.load_ext()
    lib = ctypes.CDLL(str(_build.so_path()))
    fn = lib.tmoe_route_counts_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(11)
    err = ctypes.create_string_buffer(256)
    cases = [(5000, 8, 256, 8, torch.int64), (777, 6, 64, 4, torch.int32)]
    for T, K, E, N, dt in cases:
        idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(dt)
        idx[3, 1] = -1
        idx = idx.to(dev)
        out = torch.full((E + N + 2,), -7, dtype=torch.int32, device=dev)
        stream = torch.cuda.current_stream().cuda_stream
        rc = fn(idx.data_ptr(), 1 if dt == torch.int64 else 0, T, K, E, N, out.data_ptr(), stream, err, 256)
        assert rc == 0, err.value
        torch.cuda.synchronize()
        ref = _regular_counts(idx, E, N)
        assert torch.equal(out, ref), (out.tolist()[:8], ref.tolist()[:8])
        assert torch.equal(out, _bincount_counts(idx, E, N))
        assert out[E + N + 1].item() == T and out[:E].sum().item() == T * K - 1
    # sizes beyond the built-in scratch are refused with a message, nothing is launched
    rc = fn(idx.data_ptr(), 0, 70000, 6, 64, 4, out.data_ptr(), stream, err, 256)
    assert rc == -2 and b"limits" in err.value
    rc = fn(idx.data_ptr(), 0, 100, 6, 4096, 4, out.data_ptr(), stream, err, 256)
    assert rc == -2
    # a token count near INT_MAX must be refused too (rounding it up to chunks must not wrap around)
    rc = fn(idx.data_ptr(), 0, 2 ** 31 - 1, 6, 64, 4, out.data_ptr(), stream, err, 256)
    assert rc == -2 and b"limits" in err.value
