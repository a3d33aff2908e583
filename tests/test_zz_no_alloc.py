"""Allocation-free attention backward (``mb_attn_bwd_noalloc``).

Some hosts may not allocate device memory while they run: a process that gave the whole GPU to its
own pool at start-up, or a plain C/C++ program that uses this library without PyTorch's allocator.
For them the library keeps the backward pass's fp32 work buffer in a fixed 4 MiB array inside its
own device image.  This test calls the exported C symbol directly through ``ctypes`` — as such a
host would — and checks the gradients against the regular entry point (which takes a
caller-allocated work buffer) on two consecutive calls with different inputs, so that whatever the
first call left in the shared array cannot leak into the second.  It also checks that a problem
larger than the built-in array is refused.  The file name sorts last so that a run that stops at
the first failure has already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
MB_NOALLOC_TOO_LARGE = -20


def _symbol():
    from maester_b200.ops import _lib

    lib = ctypes.CDLL(str(_lib.build()))
    fn = lib.mb_attn_bwd_noalloc
    fn.argtypes = [_P] * 10 + [_I] * 5 + [_L] * 4 + [_I, _I, _F, _P, _P]
    fn.restype = _I
    return fn


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _case(fn, seed, B, S, H, KV, hd, window):
    from maester_b200.ops import cuda as C
    from maester_b200.ops.functional import kv_block_lower_bounds, q_block_upper_bounds

    torch.manual_seed(seed)
    qkv = (torch.randn(B, S, (H + 2 * KV) * hd, device="cuda") * 0.5).to(torch.bfloat16)
    q = qkv[..., : H * hd].view(B, S, H, hd)
    k = qkv[..., H * hd:(H + KV) * hd].view(B, S, KV, hd)
    v = qkv[..., (H + KV) * hd:].view(B, S, KV, hd)
    doc = torch.zeros(B, S, dtype=torch.int32, device="cuda")
    doc[:, S // 3:] = 1
    doc[:, (2 * S) // 3:] = 2
    scale = hd ** -0.5
    lo = kv_block_lower_bounds(S, 128, window, doc, "cuda", batch=B)
    hi = q_block_upper_bounds(S, 128, window, doc, "cuda", batch=B)
    from maester_b200.ops.functional import attention_plan
    plan = attention_plan(S, window, doc, "cuda", batch=B)
    out, lse = C.attn_fwd(q, k, v, scale, True, window, plan)
    dout = torch.randn_like(out)

    want = torch.zeros(B * S, (H + 2 * KV) * hd, device="cuda", dtype=torch.bfloat16)
    C.attn_bwd(q, k, v, out, dout, lse, want, scale, True, window, plan)

    got = torch.zeros_like(want)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
            got.data_ptr(), doc.data_ptr(), lo.data_ptr(), hi.data_ptr(), B, S, H, KV, hd,
            q.stride(1), k.stride(1), v.stride(1), got.stride(0), 1, -1 if window is None else window, scale,
            status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    assert status.item() == 0
    C.check_status()
    assert _rel(got, want) < 2e-2, _rel(got, want)


def test_noalloc_matches_regular_entry_point_twice():
    fn = _symbol()
    _case(fn, 11, 2, 384, 4, 2, 128, None)   # first call on the device also does the one-time set-up
    _case(fn, 12, 1, 300, 4, 4, 256, 64)     # second call: other shapes, array still holds call 1's values


def test_noalloc_rejects_oversized_problem():
    fn = _symbol()
    # B*H*S = 2 * 64 * 16384 exceeds the 1,048,576-entry array; nothing is launched, no pointer is touched
    rc = fn(None, None, None, None, None, None, None, None, None, None, 2, 16384, 64, 8, 128,
            0, 0, 0, 0, 1, -1, 0.1, None, None)
    assert rc == MB_NOALLOC_TOO_LARGE


def test_noalloc_builtin_status_word_can_be_read_and_cleared():
    """Without a caller-provided status word the kernels report into a word inside the library;
    ``mb_noalloc_status`` reads and clears it (0 after a healthy call)."""
    from maester_b200.ops import _lib

    lib = ctypes.CDLL(str(_lib.build()))
    lib.mb_noalloc_status.restype = _I
    fn = _symbol()
    B, S, H, KV, hd = 1, 256, 2, 1, 128
    torch.manual_seed(5)
    qkv = (torch.randn(B, S, (H + 2 * KV) * hd, device="cuda") * 0.5).to(torch.bfloat16)
    q = qkv[..., : H * hd].view(B, S, H, hd)
    k = qkv[..., H * hd:(H + KV) * hd].view(B, S, KV, hd)
    v = qkv[..., (H + KV) * hd:].view(B, S, KV, hd)
    from maester_b200.ops import cuda as C
    out, lse = C.attn_fwd(q, k, v, hd ** -0.5, True, None)
    dout = torch.randn_like(out)
    got = torch.zeros(B * S, (H + 2 * KV) * hd, device="cuda", dtype=torch.bfloat16)
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
            got.data_ptr(), None, None, None, B, S, H, KV, hd, q.stride(1), k.stride(1), v.stride(1),
            got.stride(0), 1, -1, hd ** -0.5, None, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert lib.mb_noalloc_status() == 0
    assert torch.isfinite(got.float()).all() and got.float().abs().sum() > 0
