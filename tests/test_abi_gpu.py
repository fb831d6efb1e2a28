"""GPU parity tests: every kernel family is called through the nc_cuda_* C ABI (raw device pointers)
and compared with the CPU oracle on the same seeded inputs.

Tolerances (max-abs error over max-abs reference, and relative L2; both must hold):
  exact integer items (max-pool argmax, row argmax)         ==
  FP32 SIMT kernels and memory-bound kernels                2e-5   (f32 arithmetic vs double oracle)
  TF32 tensor-core contractions                             1e-3
  3xTF32 tensor-core contractions                           1e-5
"""
import ctypes as C

import numpy as np
import pytest

from oracle import nocta_oracle as O

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TOL_F32 = 2e-5
TOL_TF32 = 1e-3
TOL_3X = 1e-5
MODE_TF32, MODE_RNA, MODE_3X, MODE_SIMT = 0, 1, 2, 3


@pytest.fixture(scope="module")
def abi():
    from nocta_b200 import cuda_abi
    a = cuda_abi.load()
    assert a.nc_cuda_available(), "no CUDA device"
    a.nc_cuda_init()
    yield a
    a.nc_cuda_set_math_mode(MODE_TF32)


_keep = []


def dev(a):
    """Upload; the tensor is kept alive until the test ends, because the C ABI only sees its raw
    pointer and the caching allocator would otherwise hand the same block to the next upload."""
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    _keep.append(t)
    return t


@pytest.fixture(autouse=True)
def _release_uploads():
    yield
    torch.cuda.synchronize()
    _keep.clear()


def P(t):
    return C.c_void_p(t.data_ptr())


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


def close(got, ref, tol):
    emax, el2 = O.rel_errors(got, ref)
    assert emax <= tol and el2 <= tol, (emax, el2, tol)


def ok(abi, rc):
    assert rc == 0, abi.nc_cuda_last_message()
    assert abi.nc_cuda_device_error_word() == 0


# ------------------------------------------------------------------------------------------
# elementwise / activations
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [1, 5, 1023, 4096 + 3, 1 << 20])
def test_elementwise(abi, n):
    rng = np.random.default_rng(n)
    a = rng.standard_normal(n).astype(np.float32)
    b = (rng.standard_normal(n) + 3).astype(np.float32)
    da, db, do = dev(a), dev(b), torch.empty(n, device="cuda")
    for op, fn in enumerate([np.add, np.subtract, np.multiply, np.divide]):
        ok(abi, abi.nc_cuda_binary_f32_ex(op, P(do), P(da), P(db), n, None))
        assert np.array_equal(host(do), fn(a, b).astype(np.float32))
    ok(abi, abi.nc_cuda_scalar_f32_ex(2, P(do), P(da), 1.5, n, None))
    assert np.array_equal(host(do), a * np.float32(1.5))
    ok(abi, abi.nc_cuda_fill_f32_ex(P(do), 2.25, n, None))
    assert np.all(host(do) == 2.25)
    ok(abi, abi.nc_cuda_relu_f32_ex(P(do), P(da), n, None))
    assert np.array_equal(host(do), O.relu_forward(a))
    ok(abi, abi.nc_cuda_relu_backward_f32_ex(P(do), P(db), P(da), n, None))
    assert np.array_equal(host(do), O.relu_backward(b, a))
    ok(abi, abi.nc_cuda_gelu_f32_ex(P(do), P(da), n, None))
    close(host(do), O.gelu_forward(a), TOL_F32)
    ok(abi, abi.nc_cuda_gelu_backward_f32_ex(P(do), P(db), P(da), n, None))
    close(host(do), O.gelu_backward(b, a), TOL_F32)
    # unaligned views take the scalar path
    if n > 8:
        ok(abi, abi.nc_cuda_binary_f32_ex(0, C.c_void_p(do.data_ptr() + 4), C.c_void_p(da.data_ptr() + 4),
                                          C.c_void_p(db.data_ptr() + 4), n - 1, None))
        assert np.array_equal(host(do)[1:], (a + b)[1:])


def test_legacy_void_names(abi):
    rng = np.random.default_rng(3)
    a = rng.standard_normal(1000).astype(np.float32)
    b = rng.standard_normal(1000).astype(np.float32)
    da, db, do = dev(a), dev(b), torch.empty(1000, device="cuda")
    abi.nc_cuda_add_f32(P(do), P(da), P(db), 1000)
    assert np.array_equal(host(do), a + b)
    abi.nc_cuda_mul_scalar_f32(P(do), P(da), 0.5, 1000)
    assert np.array_equal(host(do), a * np.float32(0.5))
    bias = rng.standard_normal(10).astype(np.float32)
    abi.nc_cuda_add_broadcast_batch_f32(P(do), P(da), P(dev(bias)), 1000, 10)
    assert np.array_equal(host(do), (a.reshape(100, 10) + bias).ravel())
    assert abi.nc_cuda_last_status() == 0


def test_softmax_and_relayout(abi):
    rng = np.random.default_rng(4)
    x = (rng.standard_normal((37, 100)) * 4).astype(np.float32)
    do = torch.empty(37, 100, device="cuda")
    ok(abi, abi.nc_cuda_softmax_f32_ex(P(do), P(dev(x)), 37, 100, None))
    close(host(do), O.softmax(x), TOL_F32)
    t = rng.standard_normal((3, 5, 6, 7)).astype(np.float32)
    dn = torch.empty(3, 6, 7, 5, device="cuda")
    ok(abi, abi.nc_cuda_nchw_to_nhwc_f32_ex(P(dn), P(dev(t)), 3, 5, 42, 0, None))
    assert np.array_equal(host(dn), t.transpose(0, 2, 3, 1))
    back = torch.empty(3, 5, 6, 7, device="cuda")
    ok(abi, abi.nc_cuda_nhwc_to_nchw_f32_ex(P(back), P(dn), 3, 5, 42, None))
    assert np.array_equal(host(back), t)
    from nocta_b200.cuda_abi import size4
    # strided gather: a transposed 2-D view padded to 4 dims, and the channels-last fast path
    m = rng.standard_normal((9, 13)).astype(np.float32)
    o2 = torch.empty(13, 9, device="cuda")
    ok(abi, abi.nc_cuda_strided_copy_f32_ex(P(o2), P(dev(m)), size4([1, 1, 13, 9]), size4([0, 0, 1, 13]), None))
    assert np.array_equal(host(o2), m.T)
    o4 = torch.empty(3, 5, 6, 7, device="cuda")
    ok(abi, abi.nc_cuda_strided_copy_f32_ex(P(o4), P(dn), size4([3, 5, 6, 7]), size4([6 * 7 * 5, 1, 7 * 5, 5]), None))
    assert np.array_equal(host(o4), t)


# ------------------------------------------------------------------------------------------
# losses, reductions, optimizers
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("B,Cc", [(64, 10), (256, 100), (7, 3)])
def test_cross_entropy(abi, B, Cc):
    rng = np.random.default_rng(B)
    logits = (rng.standard_normal((B, Cc)) * 3).astype(np.float32)
    labels = rng.integers(0, Cc, B).astype(np.int64)
    if B > 8:
        labels[3] = Cc + 5  # out of range: skipped (src/ops/loss.c:278-281)
    dl, dg, dloss = dev(logits), torch.empty(B, Cc, device="cuda"), torch.zeros(1, device="cuda")
    for _ in range(2):  # second call reuses the scratch ticket
        ok(abi, abi.nc_cuda_cross_entropy_fused_f32_ex(P(dloss), P(dg), P(dl), P(dev(labels)), B, Cc, 1.0, None))
    lo, go = O.cross_entropy(logits, labels)
    close(host(dloss), lo, TOL_F32)
    close(host(dg), go, TOL_F32)


def test_mse_and_reductions(abi):
    rng = np.random.default_rng(5)
    p = rng.standard_normal((33, 129)).astype(np.float32)
    t = rng.standard_normal((33, 129)).astype(np.float32)
    dgp, dgt, dloss = torch.empty(33, 129, device="cuda"), torch.empty(33, 129, device="cuda"), torch.zeros(1, device="cuda")
    ok(abi, abi.nc_cuda_mse_fused_f32_ex(P(dloss), P(dgp), P(dgt), P(dev(p)), P(dev(t)), p.size, 1.0, None))
    lo, gp, gt = O.mse(p, t)
    close(host(dloss), lo, TOL_F32)
    close(host(dgp), gp, TOL_F32)
    close(host(dgt), gt, TOL_F32)
    x = rng.standard_normal((5, 40, 77)).astype(np.float32)
    out = torch.empty(5, 77, device="cuda")
    ok(abi, abi.nc_cuda_sum_axis_f32_ex(P(out), P(dev(x)), 5, 40, 77, None))
    close(host(out), x.astype(np.float64).sum(1), TOL_F32)
    out1 = torch.empty(200, device="cuda")
    ok(abi, abi.nc_cuda_sum_axis_f32_ex(P(out1), P(dev(x.reshape(200, 77))), 200, 77, 1, None))
    close(host(out1), x.reshape(200, 77).astype(np.float64).sum(1), TOL_F32)
    am = torch.empty(200, dtype=torch.int64, device="cuda")
    xt = x.reshape(200, 77).copy()
    xt[0, 5] = xt[0, 9] = 99.0  # tie: first index wins
    ok(abi, abi.nc_cuda_argmax_rows_f32_ex(P(am), P(dev(xt)), 200, 77, None))
    assert np.array_equal(host(am), xt.argmax(1))


@pytest.mark.parametrize("n", [7, 44426, 1 << 18])
def test_sgd_and_adam(abi, n):
    rng = np.random.default_rng(n)
    p = rng.standard_normal(n).astype(np.float32)
    dp, dv = dev(p), torch.zeros(n, device="cuda")
    cur, vel = p.copy(), None
    for step in range(3):
        g = rng.standard_normal(n).astype(np.float32)
        ok(abi, abi.nc_cuda_sgd_update_f32_ex(P(dp), P(dv), P(dev(g)), 0.01, 0.9, 0.0, 0.0, 0, int(step == 0), 1.0, n, None))
        cur, vel, _ = O.sgd_step(cur, g, vel, 0.01, momentum=0.9, first_step=(step == 0))
        close(host(dp), cur, 1e-7)
        close(host(dv), vel, 1e-7)
    # weight decay + nesterov + grad scale
    g = rng.standard_normal(n).astype(np.float32)
    dg = dev(g)
    ok(abi, abi.nc_cuda_sgd_update_f32_ex(P(dp), P(dv), P(dg), 0.01, 0.9, 0.1, 1e-3, 1, 0, 0.5, n, None))
    cur2, vel2, g2 = O.sgd_step(cur, g * np.float32(0.5), vel, 0.01, momentum=0.9, dampening=0.1, weight_decay=1e-3, nesterov=True)
    close(host(dp), cur2, 1e-7)
    close(host(dg), g2, 1e-7)
    # AdamW
    p = rng.standard_normal(n).astype(np.float32)
    dp, dm, dvv = dev(p), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    cur, m, v = p.copy(), np.zeros_like(p), np.zeros_like(p)
    for t in range(1, 4):
        g = rng.standard_normal(n).astype(np.float32)
        ok(abi, abi.nc_cuda_adam_update_f32_ex(P(dp), P(dm), P(dvv), None, P(dev(g)), 1e-3, 0.9, 0.999, 1e-8, 0.01,
                                               1 - 0.9 ** t, 1 - 0.999 ** t, 1.0, n, None))
        cur, m, v, _ = O.adam_step(cur, g, m, v, t, 1e-3, weight_decay=0.01)
        close(host(dp), cur, 1e-7)
        close(host(dm), m, 1e-7)
        close(host(dvv), v, 1e-7)


# ------------------------------------------------------------------------------------------
# pooling and normalisation (both layouts)
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("N,Cc,H,k,s", [(2, 3, 8, 2, 2), (4, 16, 12, 2, 2), (2, 8, 9, 3, 2), (2, 4, 7, 2, 1), (3, 6, 24, 2, 2)])
@pytest.mark.parametrize("layout", [0, 1])
def test_maxpool(abi, N, Cc, H, k, s, layout):
    rng = np.random.default_rng(N * 100 + H)
    x = rng.standard_normal((N, Cc, H, H)).astype(np.float32)
    x[x < 0] = 0  # ties everywhere, as after ReLU
    yo, arg = O.maxpool2d_forward(x, k, s)
    Ho = yo.shape[2]
    to_l = (lambda a: a.transpose(0, 2, 3, 1)) if layout else (lambda a: a)
    from_l = (lambda a: a.transpose(0, 3, 1, 2)) if layout else (lambda a: a)
    dx_in = dev(to_l(x))
    shape_o = (N, Ho, Ho, Cc) if layout else (N, Cc, Ho, Ho)
    dy, di = torch.empty(shape_o, device="cuda"), torch.empty(shape_o, dtype=torch.uint8, device="cuda")
    ok(abi, abi.nc_cuda_maxpool2d_forward_idx_f32_ex(P(dy), P(di), P(dx_in), N, Cc, H, H, k, s, layout, None))
    assert np.array_equal(from_l(host(dy)), yo)
    assert np.array_equal(from_l(host(di)), arg)  # bit-exact argmax offsets
    g = rng.standard_normal(yo.shape).astype(np.float32)
    dgin = torch.full(dx_in.shape, float("nan"), device="cuda")
    ok(abi, abi.nc_cuda_maxpool2d_backward_idx_f32_ex(P(dgin), P(dev(to_l(g))), P(di), N, Cc, H, H, k, s, layout, None))
    close(from_l(host(dgin)), O.maxpool2d_backward(x, g, k, s), 1e-6)
    if layout == 0:  # legacy names: forward without indices, backward recomputing the argmax
        dy2 = torch.empty(shape_o, device="cuda")
        abi.nc_cuda_maxpool2d_forward_f32(P(dy2), P(dx_in), N, Cc, H, H, k, k, s)
        assert np.array_equal(host(dy2), yo)
        dg2 = torch.full(dx_in.shape, float("nan"), device="cuda")
        abi.nc_cuda_maxpool2d_backward_f32(P(dg2), P(dev(g)), P(dx_in), None, N, Cc, H, H, k, k, s)
        close(host(dg2), O.maxpool2d_backward(x, g, k, s), 1e-6)


@pytest.mark.parametrize("N,Cc,H,W", [(4, 5, 6, 7), (8, 64, 16, 16), (2, 3, 5, 5), (16, 128, 8, 8)])
@pytest.mark.parametrize("layout", [0, 1])
def test_batchnorm(abi, N, Cc, H, W, layout):
    rng = np.random.default_rng(N + Cc)
    x = (rng.standard_normal((N, Cc, H, W)) * 2 + 3).astype(np.float32)
    gam = rng.standard_normal(Cc).astype(np.float32)
    bet = rng.standard_normal(Cc).astype(np.float32)
    rm = rng.standard_normal(Cc).astype(np.float32)
    rv = (rng.random(Cc) + 0.5).astype(np.float32)
    to_l = (lambda a: a.transpose(0, 2, 3, 1)) if layout else (lambda a: a)
    from_l = (lambda a: a.transpose(0, 3, 1, 2)) if layout else (lambda a: a)
    dx_in = dev(to_l(x))
    dy = torch.empty_like(dx_in)
    drm, drv = dev(rm), dev(rv)
    dsm, dsv = torch.empty(Cc, device="cuda"), torch.empty(Cc, device="cuda")
    ok(abi, abi.nc_cuda_batchnorm_forward_f32_ex(P(dy), P(dx_in), P(dev(gam)), P(dev(bet)), P(drm), P(drv), P(dsm), P(dsv),
                                                 N, Cc, H * W, 0.1, 1e-5, 1, layout, 0, None))
    yo, mean, var, nrm, nrv = O.batchnorm2d_forward(x, gam, bet, rm, rv, True, 0.1, 1e-5)
    close(from_l(host(dy)), yo, TOL_F32)
    close(host(dsm), mean, 1e-6)
    close(host(dsv), var, 1e-6)
    close(host(drm), nrm, 1e-6)
    close(host(drv), nrv, 1e-6)  # unbiased variance into the running buffer
    g = rng.standard_normal(x.shape).astype(np.float32)
    ddx, ddg, ddb = torch.empty_like(dx_in), torch.empty(Cc, device="cuda"), torch.empty(Cc, device="cuda")
    ok(abi, abi.nc_cuda_batchnorm_backward_f32_ex(P(ddx), P(ddg), P(ddb), P(dev(to_l(g))), P(dx_in), P(dev(gam)), P(dsm), P(dsv),
                                                  None, None, 0, N, Cc, H * W, 1e-5, layout, None))
    dxo, dgo, dbo = O.batchnorm2d_backward(g, x, gam, mean, var, 1e-5)
    close(from_l(host(ddx)), dxo, TOL_F32)
    close(host(ddg), dgo, TOL_F32)
    close(host(ddb), dbo, TOL_F32)
    # fused ReLU: forward clamps, backward masks with the forward output
    ok(abi, abi.nc_cuda_batchnorm_forward_f32_ex(P(dy), P(dx_in), P(dev(gam)), P(dev(bet)), None, None, P(dsm), P(dsv),
                                                 N, Cc, H * W, 0.1, 1e-5, 1, layout, 1, None))
    yr = O.relu_forward(yo)
    close(from_l(host(dy)), yr, TOL_F32)
    gm = np.where(from_l(host(dy)) > 0, g, 0).astype(np.float32)
    dxo, dgo, dbo = O.batchnorm2d_backward(gm, x, gam, mean, var, 1e-5)
    for relu_out, beta_p, recompute in ((P(dy), None, 0), (None, P(dev(bet)), 1)):  # mask read back / recomputed from x
        ok(abi, abi.nc_cuda_batchnorm_backward_f32_ex(P(ddx), P(ddg), P(ddb), P(dev(to_l(g))), P(dx_in), P(dev(gam)), P(dsm), P(dsv),
                                                      relu_out, beta_p, recompute, N, Cc, H * W, 1e-5, layout, None))
        close(from_l(host(ddx)), dxo, TOL_F32)
        close(host(ddg), dgo, TOL_F32)
    # eval mode (legacy name, NCHW): running statistics
    if layout == 0:
        abi.nc_cuda_batchnorm_forward_f32(P(dy), P(dx_in), P(dev(gam)), P(dev(bet)), P(drm), P(drv), P(dsm), P(dsv),
                                          N, Cc, H * W, 0.1, 1e-5, False)
        close(host(dy), O.batchnorm2d_forward(x, gam, bet, host(drm), host(drv), False)[0], TOL_F32)


@pytest.mark.parametrize("rows,cols", [(9, 24), (64, 1024), (5, 33), (300, 257)])
def test_layernorm(abi, rows, cols):
    rng = np.random.default_rng(rows)
    x = (rng.standard_normal((rows, cols)) + 1).astype(np.float32)
    gam = rng.standard_normal(cols).astype(np.float32)
    bet = rng.standard_normal(cols).astype(np.float32)
    dxin, dy = dev(x), torch.empty(rows, cols, device="cuda")
    ok(abi, abi.nc_cuda_layernorm_forward_f32_ex(P(dy), P(dxin), P(dev(gam)), P(dev(bet)), rows, cols, 1e-5, None))
    close(host(dy), O.layernorm_forward(x, gam, bet), TOL_F32)
    g = rng.standard_normal((rows, cols)).astype(np.float32)
    ddx, ddg, ddb = torch.empty(rows, cols, device="cuda"), torch.empty(cols, device="cuda"), torch.empty(cols, device="cuda")
    ok(abi, abi.nc_cuda_layernorm_backward_f32_ex(P(ddx), P(ddg), P(ddb), P(dev(g)), P(dxin), P(dev(gam)), rows, cols, 1e-5, None))
    dxo, dgo, dbo = O.layernorm_backward(g, x, gam)
    close(host(ddx), dxo, TOL_F32)
    close(host(ddg), dgo, TOL_F32)
    close(host(ddb), dbo, TOL_F32)


# ------------------------------------------------------------------------------------------
# contractions: matmul / linear / conv through both kernel families
# ------------------------------------------------------------------------------------------
MODES = [(MODE_SIMT, TOL_F32), (MODE_TF32, TOL_TF32), (MODE_RNA, TOL_TF32), (MODE_3X, TOL_3X)]


@pytest.mark.parametrize("mode,tol", MODES)
@pytest.mark.parametrize("M,N,K", [(64, 120, 256), (128, 64, 32), (256, 128, 256), (200, 100, 72), (384, 1000, 520), (1, 1, 1)])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_matmul(abi, mode, tol, M, N, K, ta, tb):
    rng = np.random.default_rng(M + N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    As = A.T.copy() if ta else A
    Bs = B.T.copy() if tb else B
    dC = torch.full((M, N), float("nan"), device="cuda")
    abi.nc_cuda_set_math_mode(mode)
    abi.nc_cuda_matmul_f32(P(dC), P(dev(As)), P(dev(Bs)), M, N, K, 1.0, 0.0, ta, tb)
    assert abi.nc_cuda_last_status() == 0, abi.nc_cuda_last_message()
    assert abi.nc_cuda_device_error_word() == 0
    close(host(dC), A.astype(np.float64) @ B.astype(np.float64), tol)


@pytest.mark.parametrize("mode,tol", MODES)
def test_matmul_alpha_beta_bias(abi, mode, tol):
    rng = np.random.default_rng(8)
    M, N, K = 256, 192, 160
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((N, K)).astype(np.float32)
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    dC = dev(C0)
    abi.nc_cuda_set_math_mode(mode)
    ok(abi, abi.nc_cuda_matmul_f32_ex(P(dC), N, P(dev(A)), K, P(dev(B)), K, M, N, K, 0.5, 2.0, 0, 1, P(dev(bias)), None))
    ref = 0.5 * (A.astype(np.float64) @ B.astype(np.float64).T) + 2.0 * C0 + bias
    close(host(dC), ref, tol)


@pytest.mark.parametrize("mode,tol", MODES)
@pytest.mark.parametrize("B,I,Oo", [(64, 256, 120), (128, 8192, 10), (256, 512, 384), (256, 1024, 100)])
def test_linear(abi, mode, tol, B, I, Oo):
    rng = np.random.default_rng(B + I)
    x = rng.standard_normal((B, I)).astype(np.float32)
    W = (rng.standard_normal((Oo, I)) / np.sqrt(I)).astype(np.float32)
    b = rng.standard_normal(Oo).astype(np.float32)
    g = rng.standard_normal((B, Oo)).astype(np.float32)
    abi.nc_cuda_set_math_mode(mode)
    dx_, dW_, db_ = dev(x), dev(W), dev(b)
    dy = torch.full((B, Oo), float("nan"), device="cuda")
    ok(abi, abi.nc_cuda_linear_forward_f32_ex(P(dy), P(dx_), P(dW_), P(db_), B, I, Oo, None))
    close(host(dy), O.linear_forward(x, W, b), tol)
    gx, gW, gb = torch.empty(B, I, device="cuda"), torch.empty(Oo, I, device="cuda"), torch.empty(Oo, device="cuda")
    ok(abi, abi.nc_cuda_linear_backward_f32_ex(P(gx), P(gW), P(gb), P(dev(g)), P(dx_), P(dW_), B, I, Oo, None))
    dxo, dWo, dbo = O.linear_backward(g, x, W)
    close(host(gx), dxo, tol)
    close(host(gW), dWo, tol)
    close(host(gb), dbo, TOL_F32)


CONV_CASES = [
    # N, Cin, H, W, Cout, k, stride, pad
    (2, 1, 12, 12, 6, 5, 1, 0),     # LeNet-like, tiny channels -> SIMT
    (2, 3, 9, 8, 5, 3, 2, 1),       # stride 2, ragged
    (2, 32, 8, 8, 32, 3, 1, 1),
    (4, 64, 14, 14, 64, 3, 1, 1),
    (2, 64, 9, 11, 96, 3, 1, 1),    # ragged image, Cout not a power of two
    (4, 128, 16, 16, 256, 3, 1, 1),
    (16, 32, 12, 12, 64, 5, 1, 2),
    (4, 3, 16, 16, 64, 3, 1, 1),    # first-layer kernels (3 input channels)
    (3, 3, 9, 11, 64, 3, 1, 1),     # 297 pixels: a ragged 128-pixel tile, an odd number of tiles
    (5, 3, 24, 40, 64, 3, 1, 0),    # no padding, 22 x 38 outputs
    (64, 3, 32, 32, 64, 3, 1, 1),   # 512 tiles: several per CTA, the rings of the tensor-core kernels wrap
    (3, 3, 9, 11, 32, 3, 1, 0),
    # shapes the halo-resident tensor-core kernels take in plain TF32 mode: whole 8-wide pixel tiles, >= 32 channels
    (2, 32, 32, 8, 32, 3, 1, 1),
    (3, 64, 32, 16, 128, 3, 1, 1),
    (2, 32, 64, 24, 48, 3, 1, 1),   # two tiles in h, three in w, Cout not a power of two
    (2, 64, 32, 8, 64, 1, 1, 0),    # 1 x 1 filter
    (2, 64, 56, 56, 64, 3, 1, 1),   # the isolated-backward benchmark's layer at a small batch (ragged in h: 56 = 32 + 24)
    (3, 128, 16, 16, 128, 3, 1, 1), # half-height tile
    (6, 256, 16, 16, 256, 3, 1, 1), # 16-row images, even batch: two images per tile, one issuing warp each
    (2, 128, 16, 24, 128, 3, 1, 1), # the same, three tiles wide
    (4, 128, 16, 12, 160, 3, 1, 1), # the same, ragged in width and in the channel tile
    (2, 64, 20, 12, 32, 3, 1, 1),   # ragged in both directions
]


@pytest.mark.parametrize("mode,tol", [(MODE_SIMT, TOL_F32), (MODE_TF32, TOL_TF32), (MODE_3X, TOL_3X)])
@pytest.mark.parametrize("case", CONV_CASES)
@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
def test_conv2d(abi, mode, tol, case, layout):
    N, Ci, H, W, Co, k, s, p = case
    rng = np.random.default_rng(sum(case))
    x = rng.standard_normal((N, Ci, H, W)).astype(np.float32)
    w = (rng.standard_normal((Co, Ci, k, k)) / np.sqrt(Ci * k * k)).astype(np.float32)
    b = rng.standard_normal(Co).astype(np.float32)
    yo = O.conv2d_forward(x, w, b, s, p)
    Ho, Wo = yo.shape[2], yo.shape[3]
    g = rng.standard_normal(yo.shape).astype(np.float32)
    dxo, dwo, dbo = O.conv2d_backward(x, w, g, s, p)
    abi.nc_cuda_set_math_mode(mode)
    from nocta_b200.cuda_abi import size4
    dw_, db_ = dev(w), dev(b)
    gw, gb = torch.full(w.shape, float("nan"), device="cuda"), torch.full((Co,), float("nan"), device="cuda")
    if layout == "nchw":
        dx_, dg_ = dev(x), dev(g)
        dy = torch.full(yo.shape, float("nan"), device="cuda")
        abi.nc_cuda_conv2d_forward_f32(P(dy), P(dx_), P(dw_), P(db_), N, Ci, H, W, Co, k, k, s, p)
        assert abi.nc_cuda_last_status() == 0, abi.nc_cuda_last_message()
        close(host(dy), yo, tol)
        gx = torch.full(x.shape, float("nan"), device="cuda")
        ok(abi, abi.nc_cuda_conv2d_backward_f32_ex(P(gx), P(gw), P(gb), P(dg_), P(dx_), P(dw_), N, Ci, H, W, Co, k, k, s, p, None))
        close(host(gx), dxo, tol)
    else:
        xs, ys = size4([H * W * Ci, 1, W * Ci, Ci]), size4([Ho * Wo * Co, 1, Wo * Co, Co])
        dx_, dg_ = dev(x.transpose(0, 2, 3, 1)), dev(g.transpose(0, 2, 3, 1))
        dy = torch.full((N, Ho, Wo, Co), float("nan"), device="cuda")
        ok(abi, abi.nc_cuda_conv2d_forward_f32_ex(P(dy), ys, P(dx_), xs, P(dw_), P(db_), N, Ci, H, W, Co, k, k, s, p, None))
        close(host(dy).transpose(0, 3, 1, 2), yo, tol)
        gx = torch.full((N, H, W, Ci), float("nan"), device="cuda")
        ok(abi, abi.nc_cuda_conv2d_backward_input_f32_ex(P(gx), xs, P(dg_), ys, P(dw_), N, Ci, H, W, Co, k, k, s, p, None))
        close(host(gx).transpose(0, 3, 1, 2), dxo, tol)
        ok(abi, abi.nc_cuda_conv2d_backward_weight_f32_ex(P(gw), P(gb), P(dg_), ys, P(dx_), xs, N, Ci, H, W, Co, k, k, s, p, None))
    close(host(gw), dwo, tol)
    close(host(gb), dbo, TOL_TF32 if (mode == MODE_TF32 and layout == "nchw") else TOL_F32)


def test_conv_known_answers(abi):
    # reference tests/test_nn.c:38-66: 2x2 ones kernel over a 3x3 ones image -> four 4.0s
    abi.nc_cuda_set_math_mode(MODE_TF32)
    y = torch.zeros(1, 1, 2, 2, device="cuda")
    abi.nc_cuda_conv2d_forward_f32(P(y), P(torch.ones(1, 1, 3, 3, device="cuda")), P(torch.ones(1, 1, 2, 2, device="cuda")),
                                   None, 1, 1, 3, 3, 1, 2, 2, 1, 0)
    assert np.all(host(y) == 4.0)
    # tests/test_ops.c:21-40: ones(2,3) x ones(3,2) -> 3.0
    c = torch.zeros(2, 2, device="cuda")
    abi.nc_cuda_matmul_f32(P(c), P(torch.ones(2, 3, device="cuda")), P(torch.ones(3, 2, device="cuda")), 2, 2, 3, 1.0, 0.0, 0, 0)
    assert np.all(host(c) == 3.0)


def test_bad_arguments_are_errors(abi):
    abi.nc_cuda_clear_status()
    assert abi.nc_cuda_relu_f32_ex(None, None, 10, None) != 0
    assert abi.nc_cuda_last_status() != 0
    abi.nc_cuda_clear_status()
    assert abi.nc_cuda_set_math_mode(99) in (0, 1, 2, 3)
    assert abi.nc_cuda_last_status() != 0
    abi.nc_cuda_clear_status()


@pytest.mark.parametrize("shape", [(3, 8, 6, 10), (2, 64, 16, 16), (5, 36, 2, 2)])
@pytest.mark.parametrize("rounding", [0, 1])
def test_fused_batchnorm_relu_maxpool_equals_the_separate_kernels(abi, shape, rounding):
    """nc_cuda_batchnorm_relu_maxpool2_*: pooled values and window offsets bit-equal to BatchNorm(+ReLU)
    followed by max-pool; gradients equal up to summation order (2e-6)."""
    N, Cc, H, W = shape
    rng = np.random.default_rng(N * 100 + Cc)
    x = dev((rng.standard_normal((N, H, W, Cc)) * 2 + 0.5).astype(np.float32))   # channels-last memory
    gamma, beta = dev(rng.standard_normal(Cc).astype(np.float32)), dev(rng.standard_normal(Cc).astype(np.float32))
    dp = dev(rng.standard_normal((N, H // 2, W // 2, Cc)).astype(np.float32))
    f32 = lambda *s: torch.empty(*s, device="cuda")
    u8 = lambda *s: torch.empty(*s, dtype=torch.uint8, device="cuda")
    prev = abi.nc_cuda_set_round_outputs(rounding)
    try:
        # separate kernels
        y, m0, v0 = f32(N, H, W, Cc), f32(Cc), f32(Cc)
        ok(abi, abi.nc_cuda_batchnorm_forward_f32_ex(P(y), P(x), P(gamma), P(beta), None, None, P(m0), P(v0), N, Cc, H * W, 0.1, 1e-5, 1, 1, 1, None))
        p0, i0 = f32(N, H // 2, W // 2, Cc), u8(N, H // 2, W // 2, Cc)
        ok(abi, abi.nc_cuda_maxpool2d_forward_idx_f32_ex(P(p0), P(i0), P(y), N, Cc, H, W, 2, 2, 1, None))
        dy, dx0, dg0, db0 = f32(N, H, W, Cc), f32(N, H, W, Cc), f32(Cc), f32(Cc)
        ok(abi, abi.nc_cuda_maxpool2d_backward_idx_f32_ex(P(dy), P(dp), P(i0), N, Cc, H, W, 2, 2, 1, None))
        ok(abi, abi.nc_cuda_batchnorm_backward_f32_ex(P(dx0), P(dg0), P(db0), P(dy), P(x), P(gamma), P(m0), P(v0), None, P(beta), 1, N, Cc, H * W, 1e-5, 1, None))
        # fused
        p1, i1, m1, v1 = f32(N, H // 2, W // 2, Cc), u8(N, H // 2, W // 2, Cc), f32(Cc), f32(Cc)
        ok(abi, abi.nc_cuda_batchnorm_relu_maxpool2_forward_f32_ex(P(p1), P(i1), P(x), P(gamma), P(beta), None, None, P(m1), P(v1), N, Cc, H, W, 0.1, 1e-5, 1, None))
        dx1, dg1, db1 = f32(N, H, W, Cc), f32(Cc), f32(Cc)
        ok(abi, abi.nc_cuda_batchnorm_relu_maxpool2_backward_f32_ex(P(dx1), P(dg1), P(db1), P(dp), P(i1), P(x), P(gamma), P(beta), P(m1), P(v1), N, Cc, H, W, 1e-5, None))
    finally:
        abi.nc_cuda_set_round_outputs(prev)
    assert torch.equal(m0, m1) and torch.equal(v0, v1)
    assert torch.equal(p0, p1)
    if rounding == 0:
        assert torch.equal(i0, i1)
        close(host(dx1), host(dx0), 2e-6)
        close(host(dg1), host(dg0), 2e-6)
        close(host(db1), host(db0), 2e-6)
    else:
        # With TF32-rounded outputs the separate pooling kernel sees rounded candidates, where two values closer than a
        # TF32 step tie and the scan order decides; the fused kernel decides on the unrounded values, as the reference
        # does.  The offsets may therefore differ, but only between candidates that are equal after rounding: the value
        # the fused offset points at in the separately computed (rounded) activation is the pooled maximum.
        win = torch.stack([y[:, 0::2, 0::2], y[:, 0::2, 1::2], y[:, 1::2, 0::2], y[:, 1::2, 1::2]], 0)
        assert torch.equal(torch.gather(win, 0, i1.long().unsqueeze(0)).squeeze(0), p1)
        assert float((i0 == i1).float().mean()) > 0.99
        if torch.equal(i0, i1):   # no tie was broken differently: the gradients follow the same routes
            close(host(dx1), host(dx0), 2e-6)
            close(host(dg1), host(dg0), 2e-6)
            close(host(db1), host(db0), 2e-6)
    # rejected shapes
    assert abi.nc_cuda_batchnorm_relu_maxpool2_forward_f32_ex(P(p1), P(i1), P(x), P(gamma), P(beta), None, None, P(m1), P(v1), N, Cc, H + 1, W, 0.1, 1e-5, 1, None) != 0
    abi.nc_cuda_clear_status()


@pytest.mark.parametrize("shape", [(8, 64, 32, 64), (4, 128, 16, 256), (6, 32, 32, 48),
                                   (8, 3, 64, 64), (5, 3, 38, 32), (3, 3, 70, 128), (4, 3, 24, 16)])  # 3 channels: the first-layer kernel
def test_batchnorm_takes_statistics_offered_by_the_convolution(abi, shape):
    """With nc_cuda_set_conv_stats(1) the forward convolution leaves per-channel sums behind and the BatchNorm
    called right after it uses them: same result (2e-6) as BatchNorm reading the tensor; the offer is void after
    any other launch or for any other tensor."""
    from nocta_b200 import cuda_abi
    N, Cin, H, Cout = shape
    rng = np.random.default_rng(Cin + Cout)
    x = dev(rng.standard_normal((N, H, H, Cin)).astype(np.float32))
    w = dev((rng.standard_normal((Cout, Cin, 3, 3)) / (3 * Cin ** 0.5)).astype(np.float32))
    b = dev(rng.standard_normal(Cout).astype(np.float32))
    gamma, beta = dev(rng.standard_normal(Cout).astype(np.float32)), dev(rng.standard_normal(Cout).astype(np.float32))
    xs = cuda_abi.size4([H * H * Cin, 1, H * Cin, Cin])
    ys = cuda_abi.size4([H * H * Cout, 1, H * Cout, Cout])
    y = torch.empty(N, H, H, Cout, device="cuda")

    def bn(inp):
        out, m, v = torch.empty_like(inp), torch.empty(Cout, device="cuda"), torch.empty(Cout, device="cuda")
        ok(abi, abi.nc_cuda_batchnorm_forward_f32_ex(P(out), P(inp), P(gamma), P(beta), None, None, P(m), P(v), N, Cout, H * H, 0.1, 1e-5, 1, 1, 1, None))
        return out, m, v

    conv = lambda: ok(abi, abi.nc_cuda_conv2d_forward_f32_ex(P(y), ys, P(x), xs, P(w), P(b), N, Cin, H, H, Cout, 3, 3, 1, 1, None))
    conv()
    ref_out, ref_m, ref_v = bn(y)                       # switch off: BatchNorm reads y
    launches_plain = abi.nc_cuda_launch_count()
    prev = abi.nc_cuda_set_conv_stats(1)
    try:
        abi.nc_cuda_reset_launch_count()
        conv()
        base = abi.nc_cuda_launch_count()
        out, m, v = bn(y)                               # takes the offer: finalize + apply only
        assert abi.nc_cuda_launch_count() - base == 2
        close(host(m), host(ref_m), 2e-6)
        close(host(v), host(ref_v), 2e-6)
        close(host(out), host(ref_out), 2e-6)
        # the offer is used once
        base = abi.nc_cuda_launch_count()
        bn(y)
        assert abi.nc_cuda_launch_count() - base == 3
        # another launch in between voids it (the tensor could have changed: here it does)
        conv()
        ok(abi, abi.nc_cuda_scalar_f32_ex(2, P(y), P(y), 2.0, y.numel(), None))   # y *= 2 in place (op 2 = mul)
        out2, m2, v2 = bn(y)
        close(host(m2), 2 * host(ref_m), 2e-6)
        # a copy into the tensor through the library voids it too
        conv()
        fresh = np.ascontiguousarray(rng.standard_normal((N, H, H, Cout)).astype(np.float32))
        abi.nc_cuda_memcpy_h2d(P(y), fresh.ctypes.data_as(C.c_void_p), fresh.nbytes)
        out3, m3, v3 = bn(y)
        close(host(m3), fresh.reshape(-1, Cout).mean(0), 2e-5)
        # and it is tied to the tensor
        conv()
        other = y.clone()
        base = abi.nc_cuda_launch_count()
        bn(other)
        assert abi.nc_cuda_launch_count() - base == 3
    finally:
        abi.nc_cuda_set_conv_stats(prev)


@pytest.mark.parametrize("shape", [(4, 128, 32, 128), (2, 128, 27, 160), (3, 256, 40, 64), (2, 160, 24, 128), (5, 128, 26, 32),
                                   (4, 256, 16, 256), (6, 128, 16, 64)])   # the last two: 16-row images, two per tile
def test_batchnorm_backward_takes_sums_from_the_input_gradient_convolution(abi, shape):
    """nc_cuda_offer_batchnorm_backward_sums_f32: the input-gradient convolution that writes the upstream gradient of a
    BatchNorm+ReLU also sums g' and g' * xhat per channel, and the BatchNorm backward called right after it skips its own
    reduction: dx, dgamma, dbeta equal the plain path (sums in another order: 2e-6 of the largest entry), the gradient the
    convolution stores is bit-identical, the offer is used once, is tied to the tensors, and any launch in between voids it."""
    from nocta_b200 import cuda_abi
    N, C, H, Cout = shape                                # C = channels of the BatchNorm = input channels of the convolution (>= 128:
                                                         # the channels-on-M kernel, the one that serves announcements)
    rng = np.random.default_rng(C * 7 + Cout)
    xbn = dev(rng.standard_normal((N, H, H, C)).astype(np.float32))             # BatchNorm input
    gamma, beta = dev(rng.standard_normal(C).astype(np.float32)), dev((0.3 * rng.standard_normal(C)).astype(np.float32))
    mean = dev(xbn.reshape(-1, C).mean(0).cpu().numpy())
    var = dev(xbn.reshape(-1, C).var(0, unbiased=False).cpu().numpy())
    w = dev((rng.standard_normal((Cout, C, 3, 3)) / (3 * C ** 0.5)).astype(np.float32))
    dy = dev(rng.standard_normal((N, H, H, Cout)).astype(np.float32))           # gradient of the convolution's output
    xs = cuda_abi.size4([H * H * C, 1, H * C, C])
    ys = cuda_abi.size4([H * H * Cout, 1, H * Cout, Cout])
    g = torch.empty(N, H, H, C, device="cuda")                                  # gradient of the convolution's input

    def offer(x_=None):
        ok(abi, abi.nc_cuda_offer_batchnorm_backward_sums_f32(P(xbn if x_ is None else x_), P(mean), P(var), P(gamma), P(beta), 1e-5, C, N * H * H))
    conv_dx = lambda: ok(abi, abi.nc_cuda_conv2d_backward_input_f32_ex(P(g), xs, P(dy), ys, P(w), N, C, H, H, Cout, 3, 3, 1, 1, None))

    def bn_bwd(grad, x_=None):
        dx, dg, db = torch.empty_like(xbn), torch.empty(C, device="cuda"), torch.empty(C, device="cuda")
        ok(abi, abi.nc_cuda_batchnorm_backward_f32_ex(P(dx), P(dg), P(db), P(grad), P(xbn if x_ is None else x_), P(gamma), P(mean), P(var), None, P(beta), 1,
                                                      N, C, H * H, 1e-5, 1, None))
        return dx, dg, db

    conv_dx()
    g_plain = g.clone()
    ref = bn_bwd(g)
    hits0 = abi.nc_cuda_batchnorm_backward_fold_count()
    abi.nc_cuda_reset_launch_count()
    offer(); conv_dx()
    assert torch.equal(g, g_plain)                        # the stored gradient does not depend on the extra sums
    base = abi.nc_cuda_launch_count()
    got = bn_bwd(g)
    assert abi.nc_cuda_batchnorm_backward_fold_count() == hits0 + 1
    assert abi.nc_cuda_launch_count() - base == 2          # finalize + apply, no reduction
    for a, b in zip(got, ref):
        close(host(a), host(b), 2e-6)
    # used once
    bn_bwd(g)
    assert abi.nc_cuda_batchnorm_backward_fold_count() == hits0 + 1
    # an announcement is consumed by the next input-gradient call only
    offer(); conv_dx(); conv_dx()
    bn_bwd(g)
    assert abi.nc_cuda_batchnorm_backward_fold_count() == hits0 + 1
    # a launch in between voids the offer (here it changes the gradient)
    offer(); conv_dx()
    ok(abi, abi.nc_cuda_scalar_f32_ex(2, P(g), P(g), 2.0, g.numel(), None))
    got2 = bn_bwd(g)
    assert abi.nc_cuda_batchnorm_backward_fold_count() == hits0 + 1
    close(host(got2[1]), 2 * host(ref[1]), 2e-6)
    # tied to the gradient tensor and to the BatchNorm's input
    offer(); conv_dx()
    bn_bwd(g.clone())
    assert abi.nc_cuda_batchnorm_backward_fold_count() == hits0 + 1
    offer(); conv_dx()
    bn_bwd(g, xbn.clone())
    assert abi.nc_cuda_batchnorm_backward_fold_count() == hits0 + 1
    # a shape the announcement does not fit is ignored by the convolution
    ok(abi, abi.nc_cuda_offer_batchnorm_backward_sums_f32(P(xbn), P(mean), P(var), P(gamma), P(beta), 1e-5, C, N * H * H + 1))
    conv_dx()
    bn_bwd(g)
    assert abi.nc_cuda_batchnorm_backward_fold_count() == hits0 + 1
    assert abi.nc_cuda_device_error_word() == 0


def test_multi_tensor_optimizer_updates_equal_the_single_tensor_kernels(abi):
    """nc_cuda_sgd_update_multi_f32_ex / nc_cuda_adam_update_multi_f32_ex: bit-equal to one call per tensor, for
    ragged sizes (1 element, not a multiple of the chunk, empty) and more tensors than one launch table holds."""
    rng = np.random.default_rng(91)
    sizes = [1, 7, 4096, 4097, 0, 100_003, 33] + [257] * 50
    mk = lambda scale=1.0: [torch.from_numpy((rng.standard_normal(n) * scale).astype(np.float32)).cuda() for n in sizes]
    p0, g0, v0, m0, s0 = mk(), mk(), mk(0.1), mk(0.1), [t.abs() for t in mk(0.01)]
    tab = lambda ts: (C.c_void_p * len(ts))(*[t.data_ptr() if t.numel() else None for t in ts])
    numel = (C.c_size_t * len(sizes))(*sizes)
    # SGD momentum + weight decay + nesterov
    pa, va = [t.clone() for t in p0], [t.clone() for t in v0]
    for p_, v_, g_ in zip(pa, va, g0):
        if p_.numel():
            ok(abi, abi.nc_cuda_sgd_update_f32_ex(P(p_), P(v_), P(g_.clone()), 0.05, 0.9, 0.1, 1e-3, 1, 0, 0.5, p_.numel(), None))
    pb, vb, gb = [t.clone() for t in p0], [t.clone() for t in v0], [t.clone() for t in g0]
    ok(abi, abi.nc_cuda_sgd_update_multi_f32_ex(len(sizes), tab(pb), tab(vb), tab(gb), numel, 0.05, 0.9, 0.1, 1e-3, 1, 0, 0.5, None))
    for a_, b_ in zip(pa + va, pb + vb):
        assert torch.equal(a_, b_)
    # AdamW
    pa, ma, sa = [t.clone() for t in p0], [t.clone() for t in m0], [t.clone() for t in s0]
    for p_, m_, s_, g_ in zip(pa, ma, sa, g0):
        if p_.numel():
            ok(abi, abi.nc_cuda_adam_update_f32_ex(P(p_), P(m_), P(s_), None, P(g_), 1e-3, 0.9, 0.999, 1e-8, 0.01, 0.1, 0.001, 1.0, p_.numel(), None))
    pb, mb, sb = [t.clone() for t in p0], [t.clone() for t in m0], [t.clone() for t in s0]
    ok(abi, abi.nc_cuda_adam_update_multi_f32_ex(len(sizes), tab(pb), tab(mb), tab(sb), None, tab(g0), numel, 1e-3, 0.9, 0.999, 1e-8, 0.01, 0.1, 0.001, 1.0, None))
    for a_, b_ in zip(pa + ma + sa, pb + mb + sb):
        assert torch.equal(a_, b_)
