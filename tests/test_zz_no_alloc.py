"""The allocation-free LSTM forward entry point against the regular one.

Some users of the library cannot allocate device memory where they run the recurrence (a host with a fixed
memory plan, a frozen allocator, a fully committed budget), so ``fbam_lstm_fwd_noalloc`` keeps the kernel's
scratch in a fixed device array inside the library.  This test calls it through its exported C symbol, twice
in a row — the array is shared and keeps the previous call's contents, so the second call checks that stale
scratch does no harm — and compares y, the cell states and the activated gates with ``fbam_lstm_fwd``.
"""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _inputs(t_len, b, h, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    k = 1.0 / math.sqrt(h)
    gates = torch.randn(t_len, b, 4 * h, device="cuda", generator=g)
    whh = ((torch.rand(4 * h, h, device="cuda", generator=g) * 2 - 1) * k).to(BF)
    h0 = 0.1 * torch.randn(h, device="cuda", generator=g)
    c0 = 0.1 * torch.randn(h, device="cuda", generator=g)
    return gates, whh, h0, c0


def _run_regular(nv, gates, whh, h0, c0, t_len, b, h):
    gates = gates.clone()
    y = torch.empty(t_len, b, h, dtype=BF, device="cuda")
    c_all = torch.empty(t_len, b, h, dtype=torch.float32, device="cuda")
    hbuf = torch.empty(2 * 8 * h, dtype=BF, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    code = nv.lib().fbam_lstm_fwd(nv.ptr(gates), nv.ptr(whh), nv.ptr(h0), nv.ptr(c0), nv.ptr(y), nv.ptr(c_all),
                                  nv.ptr(hbuf), nv.ptr(counter), nv.ptr(status), t_len, b, h, nv.stream_ptr())
    assert code == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return gates, y, c_all


def _run_noalloc(nv, gates, whh, h0, c0, t_len, b, h):
    gates = gates.clone()
    y = torch.empty(t_len, b, h, dtype=BF, device="cuda")
    c_all = torch.empty(t_len, b, h, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib = nv.lib()
    lib.fbam_lstm_fwd_noalloc.restype = C.c_int
    code = lib.fbam_lstm_fwd_noalloc(nv.ptr(gates), nv.ptr(whh), nv.ptr(h0), nv.ptr(c0), nv.ptr(y), nv.ptr(c_all),
                                     nv.ptr(status), t_len, b, h, nv.stream_ptr())
    assert code == 0, code
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return gates, y, c_all


def test_noalloc_entry_point_matches_regular_entry_point_twice():
    from fbamtrain_b200.ops import native as nv
    from fbamtrain_b200.utils.testing import assert_similar
    # two different problems back to back: the second starts from the first one's scratch contents
    for seed, (t_len, b, h) in enumerate([(24, 8, 512), (17, 3, 1024)]):
        gates, whh, h0, c0 = _inputs(t_len, b, h, seed)
        ref_g, ref_y, ref_c = _run_regular(nv, gates, whh, h0, c0, t_len, b, h)
        got_g, got_y, got_c = _run_noalloc(nv, gates, whh, h0, c0, t_len, b, h)
        # both entry points launch the same kernel on the same inputs: anything but identical bits would mean that
        # stale scratch contents leaked into the result
        assert torch.equal(ref_y, got_y), "y"
        assert torch.equal(ref_c, got_c), "c_all"
        assert torch.equal(ref_g, got_g), "gates"
        assert_similar(ref_y, got_y, 3e-2, "y")


def test_noalloc_entry_point_allocates_no_device_memory():
    """Free device memory (as the driver reports it) and this process's allocator statistics are the same before and
    after a call whose inputs and outputs already exist: the entry point takes nothing from the device heap."""
    from fbamtrain_b200.ops import native as nv
    t_len, b, h = 12, 4, 256
    gates, whh, h0, c0 = _inputs(t_len, b, h, 7)
    y = torch.empty(t_len, b, h, dtype=BF, device="cuda")
    c_all = torch.empty(t_len, b, h, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib = nv.lib()
    lib.fbam_lstm_fwd_noalloc.restype = C.c_int
    args = (nv.ptr(gates), nv.ptr(whh), nv.ptr(h0), nv.ptr(c0), nv.ptr(y), nv.ptr(c_all), nv.ptr(status), t_len, b, h,
            nv.stream_ptr())
    assert lib.fbam_lstm_fwd_noalloc(*args) == 0          # first call on the device: address look-up, module load
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    assert lib.fbam_lstm_fwd_noalloc(*args) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert torch.cuda.memory_reserved() == reserved_before
    assert int(status.item()) == 0


def test_noalloc_entry_point_rejects_oversize_with_clear_error():
    from fbamtrain_b200.ops import native as nv
    lib = nv.lib()
    lib.fbam_lstm_fwd_noalloc.restype = C.c_int
    lib.fbam_lstm_fwd_noalloc_max_hidden.restype = C.c_int
    lib.fbam_lstm_fwd_noalloc_strerror.restype = C.c_char_p
    limit = lib.fbam_lstm_fwd_noalloc_max_hidden()
    assert limit == 1024
    code = lib.fbam_lstm_fwd_noalloc(None, None, None, None, None, None, None, 4, 2, limit + 16, None)
    assert code == 401
    assert b"exceeds" in lib.fbam_lstm_fwd_noalloc_strerror(code)
