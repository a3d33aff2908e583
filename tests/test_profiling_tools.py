"""Per-launcher timers: wrapping, call counts, restoration (CPU); device times and NVTX ranges on a GPU."""
import types

import pytest
import torch


def _fake_module():
    m = types.ModuleType("fake_kernels")

    def alpha(x):
        return x + 1

    def beta(x, y=2):
        return x * y

    def _private(x):
        return x

    for f in (alpha, beta, _private):
        f.__module__ = m.__name__
        setattr(m, f.__name__, f)
    return m


def test_kernel_timers_wrap_count_and_restore():
    from maester_b200.profiling import KernelTimers
    m = _fake_module()
    orig_alpha, orig_beta = m.alpha, m.beta
    with KernelTimers(m) as kt:
        assert m.alpha is not orig_alpha and m._private.__name__ == "_private"
        assert m.alpha(1) == 2 and m.alpha(2) == 3 and m.beta(3, y=4) == 12
    assert m.alpha is orig_alpha and m.beta is orig_beta
    rep = kt.report()
    assert {k: v[0] for k, v in rep.items()} == {"alpha": 2, "beta": 1}
    assert all(v[1] >= 0.0 for v in rep.values())


def test_kernel_timers_restore_after_exception():
    from maester_b200.profiling import KernelTimers
    m = _fake_module()
    orig = m.alpha
    with pytest.raises(ZeroDivisionError):
        with KernelTimers(m):
            m.alpha(1)
            1 / 0
    assert m.alpha is orig


@pytest.mark.gpu
def test_kernel_timers_on_native_launchers():
    from maester_b200.ops import cuda as C
    from maester_b200.profiling import KernelTimers
    a = torch.randn(512, 256, device="cuda").to(torch.bfloat16)
    b = torch.randn(384, 256, device="cuda").to(torch.bfloat16)
    with KernelTimers() as kt:
        for _ in range(3):
            C.gemm(a, b)
        C.glu_fwd(torch.randn(64, 256, device="cuda").to(torch.bfloat16), 0)
    rep = kt.report()
    assert rep["gemm"][0] == 3 and rep["gemm"][1] > 0.0 and rep["glu_fwd"][0] == 1
    assert C.gemm.__name__ == "gemm"  # restored
