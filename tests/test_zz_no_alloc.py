"""GPU: fb_argmax_static (partials in a fixed in-library array) against fb_argmax.

Collected last (file name), calls the exported C symbol directly through ctypes, and runs two
calls in a row with different inputs so that the second call sees the first call's partials
still in the shared array.
"""
import ctypes

import pytest
import torch

from ferrite_b200.ops import reference as R

pytestmark = pytest.mark.gpu

MAX_ROWS = 64
E_ROWS = -2


def _symbols():
    from ferrite_b200 import _lib
    K = _lib.lib()
    f = K.lib.fb_argmax_static
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                  ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]
    s = K.lib.fb_argmax_static_strerror
    s.restype = ctypes.c_char_p
    s.argtypes = [ctypes.c_int]
    return K, f, s


def _both(K, f, logits, vocab_offset):
    n, V = logits.shape
    st = torch.cuda.current_stream().cuda_stream
    ids_a = torch.full((n,), -7, dtype=torch.int32, device="cuda")
    vals_a = torch.zeros(n, device="cuda")
    rc = f(logits.data_ptr(), V, ids_a.data_ptr(), vals_a.data_ptr(), n, V, 1, vocab_offset, st)
    assert rc == 0, rc
    ids_b = torch.full((n,), -7, dtype=torch.int32, device="cuda")
    vals_b = torch.zeros(n, device="cuda")
    part = torch.zeros(n * 64, dtype=torch.int64, device="cuda")
    K.call("fb_argmax", logits, V, part, ids_b, vals_b, n, V, 1, vocab_offset)
    torch.cuda.synchronize()
    return ids_a.cpu(), vals_a.cpu(), ids_b.cpu(), vals_b.cpu()


def test_static_argmax_matches_twice_in_a_row():
    K, f, strerror = _symbols()
    g = torch.Generator().manual_seed(5)
    # first call: many rows, a large vocabulary with a tie (first index must win)
    a = torch.randn(48, 154880, generator=g)
    a[3, 100] = a[3, 90000] = 40.0
    # second call: fewer rows and a small vocabulary, so most slices of the shared array keep
    # the first call's keys unless the kernel rewrites them
    b = torch.randn(5, 1000, generator=g)
    b[0, 999] = 30.0
    for logits, off in ((a.cuda(), 0), (b.cuda(), 1000)):
        ids_a, vals_a, ids_b, vals_b = _both(K, f, logits, off)
        assert ids_a.tolist() == ids_b.tolist()
        assert torch.equal(vals_a, vals_b)
        want = R.argmax_first(logits.float().cpu()) + off
        assert ids_a.tolist() == want.tolist()


def test_static_argmax_refuses_too_many_rows():
    K, f, strerror = _symbols()
    logits = torch.zeros(1, 64, device="cuda")
    ids = torch.full((1,), -7, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    for n in (0, MAX_ROWS + 1, 4096):
        rc = f(logits.data_ptr(), 64, ids.data_ptr(), None, n, 64, 1, 0, st)
        assert rc == E_ROWS
        assert b"64" in strerror(rc)
    torch.cuda.synchronize()
    assert ids.item() == -7  # nothing was launched
