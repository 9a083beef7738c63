"""Failure detection on the device without faulting it: every wait inside the product kernels
is bounded, and a wait that runs out reports through the sticky error word instead of hanging.
The test makes a wait run out on purpose - a barrier that nothing arrives at - with the
library's own self-test kernel, reads the status on the host, clears it, and checks that the
context is still usable by running a normal product afterwards."""
import ctypes as ct

import pytest
import torch

pytestmark = pytest.mark.gpu

QT_ERR_TIMEOUT = 7


def test_bounded_wait_runs_out_and_context_stays_usable(native_lib):
    lib = native_lib
    from optimizers import _gemm
    torch.cuda.synchronize()
    assert lib.qt_device_error(1) == 0
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = ct.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.qt_selftest_wait_timeout(ct.c_void_p(flag.data_ptr()), st) == 0
    torch.cuda.synchronize()                               # returns: the kernel gave up by itself
    assert int(flag.item()) == 1
    assert lib.qt_device_error(0) == QT_ERR_TIMEOUT        # sticky until cleared
    # while the word is set, product kernels drain without computing: the caller must clear it
    assert lib.qt_device_error(1) == QT_ERR_TIMEOUT
    assert lib.qt_device_error(0) == 0
    A = torch.randn(2, 192, 128, device="cuda")
    D, _ = _gemm.matmul(_gemm.split(A), _gemm.split(A), trans_b=True)
    torch.cuda.synchronize()
    assert lib.qt_device_error(1) == 0
    ref = A.double() @ A.double().transpose(1, 2)
    assert float((D.double() - ref).norm() / ref.norm()) < 1e-4


def test_optimizer_reports_a_device_timeout(native_lib):
    """state_dict() is a natural synchronisation point: it polls the error word and raises."""
    from optimizers.shampoo2 import ShampooAdamW
    lib = native_lib
    p = torch.nn.Parameter(torch.randn(128, 128, device="cuda"))
    opt = ShampooAdamW([p], prec_bits=4, stat_compute_steps=1, prec_compute_steps=1)
    p.grad = torch.randn_like(p)
    opt.step()
    opt.state_dict()                                       # clean run: no error
    st = ct.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.qt_selftest_wait_timeout(None, st) == 0
    with pytest.raises(RuntimeError, match="bounded device-side wait gave up"):
        opt.state_dict()
    assert lib.qt_device_error(0) == 0                     # the check clears the word after reporting
