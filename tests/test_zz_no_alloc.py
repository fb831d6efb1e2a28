"""The allocation-free cross-entropy entry point against the allocating one.

Collected last (file name) so that it also runs after every other GPU test has used the library;
it passes alone as well.  Both entry points use the same grid and the same combine order, so the
comparison is bit-exact.  Reference semantics: src/ops/loss.c:176-351.
"""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu

MAX_ROWS = 4096  # NC_CUDA_CE_STATIC_MAX_ROWS in include/nocta_cuda.h


@pytest.fixture(scope="module")
def abi():
    from nocta_b200 import cuda_abi
    return cuda_abi.load()


def P(t):
    return C.c_void_p(t.data_ptr())


def run(fn, logits, labels, scale):
    n, c = logits.shape
    loss = torch.full((1,), -1.0, device="cuda")
    grad = torch.full((n, c), 7.0, device="cuda")
    rc = fn(P(loss), P(grad), P(logits), P(labels), n, c, scale, None)
    torch.cuda.synchronize()
    return rc, loss.cpu().numpy(), grad.cpu().numpy()


@pytest.mark.parametrize("n,c", [(1, 3), (37, 10), (256, 10), (1000, 1000), (MAX_ROWS, 17)])
def test_static_matches_allocating_entry_point_twice(abi, n, c):
    g = torch.Generator().manual_seed(n * 131 + c)
    logits = (torch.randn(n, c, generator=g) * 3).cuda()
    labels = torch.randint(0, c, (n,), generator=g, dtype=torch.int64)
    if n > 4:
        labels[1] = -1      # skipped like on the reference CPU path
        labels[3] = c + 2   # out of range: skipped
    labels = labels.cuda()
    rc0, loss0, grad0 = run(abi.nc_cuda_cross_entropy_fused_f32_ex, logits, labels, 0.5)
    assert rc0 == 0
    for _ in range(2):  # two calls in a row share the fixed scratch
        rc, loss, grad = run(abi.nc_cuda_cross_entropy_fused_static_f32_ex, logits, labels, 0.5)
        assert rc == 0
        assert np.array_equal(loss.view(np.uint32), loss0.view(np.uint32))
        assert np.array_equal(grad.view(np.uint32), grad0.view(np.uint32))
    # and against float64 numpy
    x = logits.cpu().numpy().astype(np.float64)
    lab = labels.cpu().numpy()
    m = x.max(1, keepdims=True)
    lse = np.log(np.exp(x - m).sum(1)) + m[:, 0]
    valid = (lab >= 0) & (lab < c)
    ref = (lse[valid] - x[np.nonzero(valid)[0], lab[valid]]).sum() / n
    assert abs(float(loss0[0]) - ref) <= 2e-6 * max(1.0, abs(ref))


def test_loss_only_and_grad_only(abi):
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(64, 12, generator=g).cuda()
    labels = torch.randint(0, 12, (64,), generator=g, dtype=torch.int64).cuda()
    _, loss0, grad0 = run(abi.nc_cuda_cross_entropy_fused_f32_ex, logits, labels, 1.0)
    loss = torch.zeros(1, device="cuda")
    assert abi.nc_cuda_cross_entropy_fused_static_f32_ex(P(loss), None, P(logits), P(labels), 64, 12, 1.0, None) == 0
    grad = torch.zeros(64, 12, device="cuda")
    assert abi.nc_cuda_cross_entropy_fused_static_f32_ex(None, P(grad), P(logits), P(labels), 64, 12, 1.0, None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(loss.cpu().numpy(), loss0)
    assert np.array_equal(grad.cpu().numpy(), grad0)


def test_rejects_more_rows_than_the_fixed_scratch_holds(abi):
    n, c = MAX_ROWS + 1, 4
    logits = torch.zeros(n, c, device="cuda")
    labels = torch.zeros(n, dtype=torch.int64, device="cuda")
    loss = torch.full((1,), -1.0, device="cuda")
    rc = abi.nc_cuda_cross_entropy_fused_static_f32_ex(P(loss), None, P(logits), P(labels), n, c, 1.0, None)
    torch.cuda.synchronize()
    assert rc == 5   # "request exceeds a stated fixed capacity"
    abi.lib.nc_cuda_last_message.restype = C.c_char_p
    assert b"at most 4096 rows" in abi.lib.nc_cuda_last_message()
    assert float(loss.cpu()[0]) == -1.0  # nothing was launched
    # the library stays usable
    rc = abi.nc_cuda_cross_entropy_fused_static_f32_ex(P(loss), None, P(logits[:8]), P(labels[:8]), 8, c, 1.0, None)
    torch.cuda.synchronize()
    assert rc == 0 and abs(float(loss.cpu()[0]) - np.log(4.0)) < 1e-6


def test_static_entry_point_leaves_device_memory_untouched(abi):
    """The property the entry point exists for: once its inputs and outputs exist, calling it allocates nothing on the
    device.  After one call (which resolves the scratch address on this device) the free-memory figure of cudaMemGetInfo
    must stay exactly where it was across calls of every size up to the limit, new streams included."""
    sizes = [(1, 3), (300, 100), (2048, 10), (MAX_ROWS, 64)]
    g = torch.Generator().manual_seed(9)
    cases = []
    for n, c in sizes:   # every buffer the calls will touch is created first (and kept alive)
        cases.append((torch.randn(n, c, generator=g).cuda(), torch.randint(0, c, (n,), generator=g, dtype=torch.int64).cuda(),
                      torch.zeros(1, device="cuda"), torch.zeros(n, c, device="cuda"), n, c))
    side = torch.cuda.Stream()
    logits, labels, loss, grad, n, c = cases[0]
    assert abi.nc_cuda_cross_entropy_fused_static_f32_ex(P(loss), P(grad), P(logits), P(labels), n, c, 1.0, None) == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        for logits, labels, loss, grad, n, c in cases:
            assert abi.nc_cuda_cross_entropy_fused_static_f32_ex(P(loss), P(grad), P(logits), P(labels), n, c, 1.0, None) == 0
            torch.cuda.synchronize()
            assert abi.nc_cuda_cross_entropy_fused_static_f32_ex(P(loss), None, P(logits), P(labels), n, c, 1.0, C.c_void_p(side.cuda_stream)) == 0
            torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)
