"""The tensor-core matrix product alone, against float64, at many shapes."""
import math

import numpy as np
import pytest
import torch

import plain_gptj as P
from qstream_b200.csrc import gemm_tc

pytestmark = pytest.mark.gpu


def f64(t):
    return t.detach().cpu().to(torch.float64).numpy()


SHAPES = [(1, 128, 64), (1, 4096, 4096), (3, 200, 96), (8, 320, 320), (16, 64, 256), (17, 136, 72),
          (33, 500, 1024), (64, 256, 64), (65, 256, 64), (128, 128, 128), (200, 330, 520), (256, 384, 2048),
          (1000, 96, 320), (2048, 512, 4096),
          # CTA pairs: token counts and widths just past a tile border, widths that are no multiple of 256
          (129, 136, 64), (257, 520, 136), (383, 1000, 192), (640, 1288, 72),
          # CTA pairs: more tiles than pairs, with and without a whole round of them
          (1000, 1288, 4096), (2048, 4096, 1024), (300, 9000, 1536),
          # more than 2,048 tokens: tiles walked in groups of rows (here groups of 1, 3 and 16 pairs of row tiles)
          (2304, 520, 40960), (2560, 1000, 20480), (4352, 264, 4096),
          # few tokens: tiles of 88, 112 and 120 rows, a last tile that reaches past N, more tiles than SMs
          (8, 12288, 256), (64, 16384, 128), (4, 50400, 128), (40, 2104, 320), (2, 19000, 64),
          # 65 to 128 tokens still stream the weights (128 tokens on the N side), with and without cuts along K
          (100, 12288, 256), (128, 2104, 320), (96, 520, 16384), (127, 4096, 4096)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_plain_product(M, N, K):
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().cuda()
    assert gemm_tc.takes(x, w)
    got = gemm_tc.linear(x, w, out_dtype=torch.float32)
    gemm_tc.check_status(x.device)
    ref = f64(x) @ f64(w).T
    np.testing.assert_allclose(f64(got), ref, atol=2e-3, rtol=2e-3)   # float32 accumulation of exact products


@pytest.mark.parametrize("M", [5, 40, 100, 300])
@pytest.mark.parametrize("act", [None, "gelu_new", "gelu"])
def test_epilogue(M, act):
    N, K = 264, 136
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, K, generator=g).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().cuda()
    bias = torch.randn(N, generator=g).bfloat16().cuda()
    r1 = torch.randn(M, N, generator=g).bfloat16().cuda()
    r2 = torch.randn(M, N, generator=g).bfloat16().cuda()
    fn = {None: lambda u: u, "gelu_new": P.gelu_new, "gelu": P.gelu_erf}[act]
    ref = fn(f64(x) @ f64(w).T + f64(bias)) + f64(r1) + f64(r2)
    got32 = gemm_tc.linear(x, w, bias, act, (r1, r2), torch.float32)
    np.testing.assert_allclose(f64(got32), ref, atol=3e-3, rtol=3e-3)
    got16 = gemm_tc.linear(x, w, bias, act, (r1, r2))
    assert got16.dtype == torch.bfloat16
    np.testing.assert_allclose(f64(got16), ref, atol=3e-2, rtol=1e-2)
    fbias = bias.float()
    got = gemm_tc.linear(x, w, fbias, act, (), torch.float32)
    np.testing.assert_allclose(f64(got), fn(f64(x) @ f64(w).T + f64(bias)), atol=3e-3, rtol=3e-3)
    gemm_tc.check_status(x.device)


def test_strided_input_and_row_independence():
    g = torch.Generator().manual_seed(3)
    buf = torch.randn(90, 3 * 128, generator=g).bfloat16().cuda()
    x = buf[:, 128:256]                                   # a column slice: row stride 384
    w = (torch.randn(200, 128, generator=g) / 11).bfloat16().cuda()
    assert gemm_tc.takes(x, w)
    whole = gemm_tc.linear(x, w, out_dtype=torch.float32)
    np.testing.assert_allclose(f64(whole), f64(x) @ f64(w).T, atol=2e-3, rtol=2e-3)
    # one row's result is the same bits in a batch of 90 (tokens on the M side) and of 2, 20, 50
    # (tokens on the N side): one TMEM cell per element, products summed in ascending k (K is too
    # short here for split-K)
    for rows in (slice(7, 9), slice(10, 30), slice(40, 90)):
        part = gemm_tc.linear(x[rows], w, out_dtype=torch.float32)
        assert torch.equal(part, whole[rows])
    gemm_tc.check_status(x.device)


@pytest.mark.parametrize("N,K", [(256, 4096), (4096, 4096), (520, 16384), (12288, 1024), (12288, 4096), (1192, 2048)])
def test_split_k_is_exact_and_does_not_depend_on_the_batch(N, K):
    """Few tokens and a long K: the product is cut along K over several CTAs whose partial tiles are
    added in slice order.  The result must match float64, be the same bits on every call, and a
    token's row must not depend on how many other tokens came with it."""
    g = torch.Generator().manual_seed(N + K)
    x = torch.randn(64, K, generator=g).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().cuda()
    bias = torch.randn(N, generator=g).bfloat16().cuda()
    res = torch.randn(64, N, generator=g).bfloat16().cuda()
    whole = gemm_tc.linear(x, w, bias, "gelu_new", (res,), torch.float32)
    ref = P.gelu_new(f64(x) @ f64(w).T + f64(bias)) + f64(res)
    np.testing.assert_allclose(f64(whole), ref, atol=3e-3, rtol=3e-3)
    for _ in range(3):
        assert torch.equal(gemm_tc.linear(x, w, bias, "gelu_new", (res,), torch.float32), whole)
    for rows in (slice(0, 1), slice(5, 13), slice(30, 62), slice(3, 40)):
        part = gemm_tc.linear(x[rows], w, bias, "gelu_new", (res[rows],), torch.float32)
        assert torch.equal(part, whole[rows]), rows
    gemm_tc.check_status(x.device)


@pytest.mark.parametrize("M,N,K", [(256, 4096, 20480), (512, 4096, 20480), (300, 520, 16384), (700, 1000, 8192),
                                   (129, 256, 2048), (400, 4096, 4096)])
def test_cta_pairs_cut_along_k(M, N, K):
    """A few hundred tokens against a narrow N give fewer tiles than CTA pairs: the tiles' k-ranges are cut
    for the idle pairs, the parts meet in a workspace and the last to arrive adds them in order and runs the
    epilogue.  Against float64, with bias, activation and residual; the same bits on every call."""
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().cuda()
    bias = torch.randn(N, generator=g).bfloat16().cuda()
    res = torch.randn(M, N, generator=g).bfloat16().cuda()
    ref = P.gelu_new(f64(x) @ f64(w).T + f64(bias)) + f64(res)
    got = gemm_tc.linear(x, w, bias, "gelu_new", (res,), torch.float32)
    np.testing.assert_allclose(f64(got), ref, atol=3e-3, rtol=3e-3)
    for _ in range(3):
        assert torch.equal(gemm_tc.linear(x, w, bias, "gelu_new", (res,), torch.float32), got)
    got16 = gemm_tc.linear(x, w, bias, "gelu_new", (res,))
    np.testing.assert_allclose(f64(got16), ref, atol=3e-2, rtol=1e-2)
    plain = gemm_tc.linear(x, w, out_dtype=torch.float32)
    np.testing.assert_allclose(f64(plain), f64(x) @ f64(w).T, atol=2e-3, rtol=2e-3)
    gemm_tc.check_status(x.device)


@pytest.mark.parametrize("M", [1, 8, 64, 100, 300, 1000])
def test_matrix_as_columns_of_a_wider_one(M):
    """The matrix may be a range of columns of a wider one (row stride beyond K), as the two halves of a
    block's fused output matrix are: the same bits as with a copy of those columns, in every arrangement
    of the kernel (weights streamed, tiles, CTA pairs)."""
    g = torch.Generator().manual_seed(M)
    wide = (torch.randn(520, 1024 + 2048, generator=g) / 40).bfloat16().cuda()
    bias = torch.randn(520, generator=g).float().cuda()
    for lo, hi in ((0, 1024), (1024, 3072), (8, 3064)):
        x = torch.randn(M, hi - lo, generator=g).bfloat16().cuda()
        res = torch.randn(M, 520, generator=g).bfloat16().cuda()
        view = wide[:, lo:hi]
        assert not view.is_contiguous() and gemm_tc.takes(x, view)
        got = gemm_tc.linear(x, view, bias, "gelu", (res,), torch.float32)
        assert torch.equal(got, gemm_tc.linear(x, view.contiguous(), bias, "gelu", (res,), torch.float32))
        ref = P.gelu_erf(f64(x) @ f64(view).T + f64(bias)) + f64(res)
        np.testing.assert_allclose(f64(got), ref, atol=3e-3, rtol=3e-3)
    assert not gemm_tc.takes(x, wide[:, 4:1028])          # a view that starts off a 16-byte boundary
    assert not gemm_tc.takes(x, wide.T)
    gemm_tc.check_status(x.device)
