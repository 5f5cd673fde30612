"""
The allocation-free pointwise convolution (ios_pointwise_conv_static_scratch), called through the
C-ABI with device pointers.  It exists for callers that cannot allocate device memory when they
need a convolution (a plug-in living inside another framework's pool, a loop that must not touch
the allocator): its split-K scratch is a fixed array in the library image.  The test runs it twice
in a row on the shared scratch -- with different split factors, so the second call meets the first
call's leftovers -- and compares each result with the arena-backed single-pass entry point
(ios_conv2d, impl 3) and with the CPU oracle within the TF32 tolerance of the suite.  A caller of
this entry point cannot see a device-side time-out from its return value (the call does not wait),
so the tests also read it back through ios_static_scratch_status.  Collected last on purpose.
"""
import ctypes

import numpy as np
import pytest

from ios.contrib import ios_runtime as rt
from helpers import TOL_TF32
import ios_oracle as oracle

pytestmark = pytest.mark.gpu


def _entry():
    lib = rt.load_ios_library()
    fn = lib.ios_pointwise_conv_static_scratch
    fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 5 + [ctypes.c_void_p]
    fn.restype = ctypes.c_int
    lib.ios_static_scratch_status.argtypes = [ctypes.c_void_p]
    lib.ios_static_scratch_status.restype = ctypes.c_int
    return lib, fn


def test_static_scratch_conv_matches_arena_backed_conv_twice():
    import torch
    lib, fn = _entry()
    n, h, w, cin, cout = 2, 9, 11, 160, 72
    pixels = n * h * w
    rng = np.random.default_rng(0)
    for call, (split, act) in enumerate(((5, 1), (2, 0))):
        x = rng.standard_normal((n, cin, h, w)).astype(np.float32)
        wt = (rng.standard_normal((cout, cin, 1, 1)) / np.sqrt(cin)).astype(np.float32)
        b = (rng.standard_normal(cout) * 0.1).astype(np.float32)
        expect = rt.conv2d(x, wt, b, act=('identity', 'relu')[act], impl='tensor1')      # existing entry point
        x_dev = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()   # NHWC
        w_dev = torch.from_numpy(wt.reshape(cout, cin)).cuda()
        b_dev = torch.from_numpy(b).cuda()
        y_dev = torch.full((pixels, cout), float('nan'), dtype=torch.float32, device='cuda')
        torch.cuda.synchronize()
        status = fn(x_dev.data_ptr(), w_dev.data_ptr(), b_dev.data_ptr(), y_dev.data_ptr(), pixels, cin, cout, act,
                    split, None)
        assert status == 0, lib.ios_last_error().decode()
        assert lib.ios_static_scratch_status(None) == 0, lib.ios_last_error().decode()   # waits, then reads the time-out word
        got = y_dev.cpu().numpy().reshape(n, h, w, cout).transpose(0, 3, 1, 2)
        assert np.isfinite(got).all()
        err = oracle.max_rel_err(got, expect)
        assert err <= TOL_TF32, f'call {call}: {err:.3e}'
        ref = oracle.conv2d_numpy(x, wt, b, (1, 1), (0, 0), 1, ('identity', 'relu')[act])
        assert oracle.max_rel_err(got, ref) <= TOL_TF32


@pytest.mark.parametrize('cout,split,offset', [
    (72, 0, 0),      # automatic split
    (70, 3, 0),      # cout % 4 != 0: results leave through plain stores
    (37, 0, 0),      # odd cout, automatic split
    (64, 4, 1),      # y not 16-byte aligned: plain stores again
])
def test_static_scratch_conv_against_the_oracle(cout, split, offset):
    import torch
    lib, fn = _entry()
    n, h, w, cin = 1, 17, 17, 192
    pixels = n * h * w
    rng = np.random.default_rng(cout + split)

    def tf32(a):
        """Keep the 10 mantissa bits a TF32 operand has: the tensor core then multiplies exactly what the oracle does."""
        return (a.astype(np.float32).view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)

    # this entry point takes the caller's weights as they are (nothing is packed or rounded on the way in), so the
    # tensor core drops the low 13 bits of both operands; with operands that have none, only the order of the
    # fp32 additions differs from the oracle
    x = tf32(rng.standard_normal((n, cin, h, w)))
    wt = tf32(rng.standard_normal((cout, cin, 1, 1)) / np.sqrt(cin))
    b = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    ref = oracle.conv2d_numpy(x, wt, b, (1, 1), (0, 0), 1, 'tanh')
    x_dev = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 3, 1))).cuda()
    w_dev = torch.from_numpy(wt.reshape(cout, cin)).cuda()
    b_dev = torch.from_numpy(b).cuda()
    y_all = torch.full((pixels * cout + 4,), float('nan'), dtype=torch.float32, device='cuda')
    y_dev = y_all[offset:offset + pixels * cout]
    torch.cuda.synchronize()
    for _ in range(2):
        status = fn(x_dev.data_ptr(), w_dev.data_ptr(), b_dev.data_ptr(), y_dev.data_ptr(), pixels, cin, cout, 3, split, None)
        assert status == 0, lib.ios_last_error().decode()
        assert lib.ios_static_scratch_status(None) == 0, lib.ios_last_error().decode()
        got = y_dev.cpu().numpy().reshape(n, h, w, cout).transpose(0, 3, 1, 2)
        assert oracle.max_rel_err(got, ref) <= 2e-5
    assert torch.isnan(y_all[offset + pixels * cout:]).all()          # nothing was written past the output


def test_static_scratch_conv_refuses_what_does_not_fit():
    import torch
    lib, fn = _entry()
    x = torch.zeros(16, device='cuda')
    # 2,000,000 pixels x 256 channels split 8 ways needs far more than the 8 MiB of static scratch
    assert fn(x.data_ptr(), x.data_ptr(), None, x.data_ptr(), 2000000, 64, 256, 0, 8, None) == 6
    assert b'static scratch' in lib.ios_last_error()
    assert fn(x.data_ptr(), x.data_ptr(), None, x.data_ptr(), 100, 6, 8, 0, 1, None) == 3       # cin % 4 != 0
    assert fn(None, x.data_ptr(), None, x.data_ptr(), 100, 8, 8, 0, 1, None) == 3
