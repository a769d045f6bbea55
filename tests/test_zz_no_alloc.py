"""The allocation-free product entry point, fc_qmatmul_dev_noalloc, against fc_qmatmul_dev.

Who needs it: a caller that is inside a CUDA stream capture, one that runs under a device-memory plan
that was approved up front and must not grow, or a serving loop that cannot take the device-wide stall
a cudaMalloc brings. Such a caller hands in its own x and y buffers and the library keeps its one piece
of scratch (the fp16 copy of x) in a fixed array of its device image, so nothing is allocated.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test. It must pass alone in a fresh process and after the rest of the suite; it makes two calls
in a row because the scratch is shared and keeps the previous call's contents.
"""
import ctypes as C

import numpy as np
import pytest

from ferrum_gpu_b200 import Mode, QKind, upload_quantised
from ferrum_gpu_b200 import _ffi

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", [QKind.Q4_0, QKind.Q8_0])
def test_no_alloc_product_matches_the_allocating_one_twice_in_a_row(dev, kind):
    import torch
    from oracle import oracle as orc
    lib = _ffi.load()
    k, n = 768, 520
    rng = np.random.default_rng(21)
    w = (rng.standard_normal(k * n, dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    qw = upload_quantised(dev, kind, w, k, n)
    w_deq = orc.snap_matrix(int(kind), w, k, n)  # [k, n], the values the kernels multiply with
    # the second call is smaller than the first, so stale scratch beyond its m * k elements is present
    for m, seed in ((300, 1), (77, 2)):
        x = torch.from_numpy(np.random.default_rng(seed).standard_normal((m, k), dtype=np.float32)).cuda()
        y_ref = torch.zeros(m, n, dtype=torch.float32, device="cuda")
        y_new = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        dev.check(lib.fc_qmatmul_dev(qw.handle, x.data_ptr(), m, y_ref.data_ptr(), int(Mode.TENSOR_F16)))
        dev.sync()
        dev.check(lib.fc_qmatmul_dev_noalloc(qw.handle, x.data_ptr(), m, y_new.data_ptr()))
        dev.sync()
        a, b = y_ref.cpu().numpy(), y_new.cpu().numpy()
        assert np.isfinite(b).all()
        # same kernels on the same fp16 copy: the tolerance of the tensor path (2e-2) is far from needed
        assert np.abs(a - b).max() <= 2e-2
        assert np.array_equal(a, b)
        # and against the CPU oracle over the dequantised weights, at the tensor path's bound
        want = orc.matmul(x.cpu().numpy(), w_deq, m, k, n).reshape(m, n)
        assert np.abs(b - want).max() <= 2e-2
    # nothing is allocated: device memory does not move over calls of growing size, on a weight that has only
    # ever been used through this entry point (no fp16 buffer of its own was ever made for it)
    fresh = upload_quantised(dev, kind, w, k, n)
    xs = torch.randn(512, k, device="cuda")
    ys = torch.empty(512, n, device="cuda")
    dev.check(lib.fc_qmatmul_dev_noalloc(fresh.handle, xs.data_ptr(), 8, ys.data_ptr()))
    dev.sync()
    free0 = torch.cuda.mem_get_info()[0]
    for rows in (16, 64, 200, 512):
        dev.check(lib.fc_qmatmul_dev_noalloc(fresh.handle, xs.data_ptr(), rows, ys.data_ptr()))
    dev.sync()
    assert torch.cuda.mem_get_info()[0] == free0
    # a pointer into the middle of a buffer (4-byte but not 16-byte aligned) is refused before any launch
    before = dev.launch_count()
    assert lib.fc_qmatmul_dev_noalloc(fresh.handle, xs.data_ptr() + 4, 8, ys.data_ptr()) == _ffi.FC_ERR_ARG
    assert lib.fc_qmatmul_dev(fresh.handle, xs.data_ptr(), 8, ys.data_ptr() + 4, int(Mode.TENSOR_F16)) == _ffi.FC_ERR_ARG
    assert dev.launch_count() == before and b"16-byte aligned" in lib.fc_last_error(dev.handle)
    fresh.close()
    # a product larger than the fixed scratch is refused, with a message, before anything is launched
    big_m = (4 << 20) // k + 1
    before = dev.launch_count()
    rc = lib.fc_qmatmul_dev_noalloc(qw.handle, x.data_ptr(), big_m, y_new.data_ptr())
    assert rc == _ffi.FC_ERR_SHAPE and dev.launch_count() == before
    assert b"fixed scratch" in lib.fc_last_error(dev.handle)
    qw.close()

