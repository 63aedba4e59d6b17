"""The allocation-free decode attention entry point, called through its exported C symbol.

Some callers of the kernel library cannot allocate device memory: they run inside a fixed
memory plan, as a guest in a process whose allocator is not theirs, or in a region where
cudaMalloc is forbidden.  For them `qs_attention_decode_static` keeps the scratch for the key
splits in an array inside the library.  This test calls it twice in a row and compares each
result with the ordinary entry point's, which takes the scratch from the caller (the same
kernels on the same inputs: the results must be equal bit for bit) and with plain attention in
float64; it also checks that a call beyond the array's size is refused and that a position
outside the stated bound is reported through the status word without any access.  It lives in a file that pytest
collects last, so a run that stops at the first failure has run everything else first.
"""
import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ARGS = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
        c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int]


def _library():
    from qstream_b200.csrc import build
    lib = ctypes.CDLL(str(build.build()))
    lib.qs_attention_decode_static.argtypes = ARGS + [c_void_p, c_void_p]
    lib.qs_attention_decode_static.restype = c_int
    lib.qs_attention_decode.argtypes = ARGS + [c_void_p, c_void_p, c_void_p]
    lib.qs_attention_decode.restype = c_int
    lib.qs_attention_decode_scratch.argtypes = [c_int, c_int, c_int, c_int]
    lib.qs_attention_decode_scratch.restype = c_longlong
    lib.qs_last_error.restype = ctypes.c_char_p
    return lib


def _case(seed, lens, H, dh, n_pages=40):
    g = torch.Generator().manual_seed(seed)
    pt, max_pages = 64, 8
    k_cache = torch.randn(n_pages, H, pt, dh, generator=g).bfloat16().cuda()
    v_cache = torch.randn(n_pages, H, pt, dh, generator=g).bfloat16().cuda()
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((len(lens), max_pages), -1, dtype=torch.int32)
    for s, n in enumerate(lens):
        for i in range(-(-n // pt)):
            table[s, i] = perm.pop()
    q = torch.randn(len(lens), H * dh, generator=g).bfloat16().cuda()
    slot = torch.arange(len(lens), dtype=torch.int32).cuda()
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda()
    return q, k_cache, v_cache, table.cuda(), slot, pos


def test_static_scratch_matches_caller_scratch_twice():
    lib = _library()
    H, dh, ctx = 4, 64, 4096
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32).cuda()
    for call, lens in enumerate(([300, 17, 512], [64, 450])):        # the second call reuses the array as the first left it
        q, kc, vc, table, slot, pos = _case(call, lens, H, dh)
        T = len(lens)
        common = [q.data_ptr(), H * dh, kc.data_ptr(), vc.data_ptr(), table.data_ptr(), table.shape[1], 64,
                  slot.data_ptr(), pos.data_ptr(), T, H, H, dh, dh ** -0.5, 0, ctx]
        want = torch.empty(T, H * dh, dtype=torch.bfloat16).cuda()
        scratch = torch.empty(lib.qs_attention_decode_scratch(T, H, dh, ctx), dtype=torch.float32).cuda()
        rc = lib.qs_attention_decode(want.data_ptr(), H * dh, *common, scratch.data_ptr(), status.data_ptr(), stream)
        assert rc == 0, lib.qs_last_error()
        got = torch.full((T, H * dh), float("nan"), dtype=torch.bfloat16).cuda()
        rc = lib.qs_attention_decode_static(got.data_ptr(), H * dh, *common, status.data_ptr(), stream)
        assert rc == 0, lib.qs_last_error()
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(got, want)
        np.testing.assert_allclose(got.float().cpu().numpy(), _plain(q, kc, vc, table, lens, H, dh), atol=2e-2, rtol=2e-2)


def _plain(q, kc, vc, table, lens, H, dh):
    """softmax(q.k / sqrt(dh)) v over each sequence's keys, float64, from the pages its table row names."""
    out = np.zeros((len(lens), H * dh))
    kc, vc, q, table = kc.float().cpu().numpy().astype(np.float64), vc.float().cpu().numpy().astype(np.float64), \
        q.float().cpu().numpy().astype(np.float64), table.cpu().numpy()
    for s, n in enumerate(lens):
        pages = table[s, :-(-n // 64)]
        for h in range(H):
            k = kc[pages, h].reshape(-1, dh)[:n]
            v = vc[pages, h].reshape(-1, dh)[:n]
            sc = k @ q[s, h * dh:(h + 1) * dh] / np.sqrt(dh)
            w = np.exp(sc - sc.max())
            out[s, h * dh:(h + 1) * dh] = (w / w.sum()) @ v
    return out


def test_a_position_outside_the_bound_is_reported_not_read():
    """`tok_pos` must lie below max_context rounded up to 256: a larger one sets status 1, gives a row of
    zeros and touches neither the cache nor the scratch beyond the call's share."""
    lib = _library()
    H, dh, ctx = 4, 64, 4096
    q, kc, vc, table, slot, pos = _case(9, [100, 200], H, dh)
    pos[1] = 5000
    out = torch.full((2, H * dh), float("nan"), dtype=torch.bfloat16).cuda()
    status = torch.zeros(1, dtype=torch.int32).cuda()
    rc = lib.qs_attention_decode_static(out.data_ptr(), H * dh, q.data_ptr(), H * dh, kc.data_ptr(), vc.data_ptr(),
                                        table.data_ptr(), table.shape[1], 64, slot.data_ptr(), pos.data_ptr(),
                                        2, H, H, dh, dh ** -0.5, 0, ctx, status.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.qs_last_error()
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    assert (out[1].float() == 0).all()
    np.testing.assert_allclose(out[:1].float().cpu().numpy(), _plain(q, kc, vc, table, [100], H, dh), atol=2e-2, rtol=2e-2)


def test_static_scratch_refuses_what_does_not_fit():
    lib = _library()
    H, dh = 4, 64
    q, kc, vc, table, slot, pos = _case(5, [10], H, dh)
    out = torch.empty(1, H * dh, dtype=torch.bfloat16).cuda()
    status = torch.zeros(1, dtype=torch.int32).cuda()
    rc = lib.qs_attention_decode_static(out.data_ptr(), H * dh, q.data_ptr(), H * dh, kc.data_ptr(), vc.data_ptr(),
                                        table.data_ptr(), table.shape[1], 64, slot.data_ptr(), pos.data_ptr(),
                                        1, H, H, dh, dh ** -0.5, 0, 1 << 24, status.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream)
    assert rc == 11 and b"scratch" in lib.qs_last_error()
