"""pd_softmax_ce_fwd_static: the criterion forward for callers that cannot allocate device memory
(a stage with a fixed HBM plan, or a host runtime that forbids cudaMalloc once training runs).
It keeps its per-row scratch in an array inside the library; this test calls it through the C-ABI
twice in a row and checks it against pd_softmax_ce_fwd, which takes the scratch from the caller.
Collected last on purpose: a failure here cannot hide a failure of any other test under `-x`."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

from pipedream_b200 import _lib  # noqa: E402
from pipedream_b200._lib import call  # noqa: E402


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _both(logits, target, smoothing, padding_idx, scale):
    rows, C = logits.shape
    dt = 1 if logits.dtype == torch.bfloat16 else 0
    s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    row_loss = torch.empty(rows, device="cuda")
    lse_a, loss_a = torch.empty(rows, device="cuda"), torch.empty((), device="cuda")
    call("pd_softmax_ce_fwd", _p(logits), dt, _p(target), rows, C, smoothing, padding_idx, scale, _p(row_loss),
         _p(lse_a), _p(loss_a), s)
    lse_b, loss_b = torch.full((rows,), -1.0, device="cuda"), torch.full((), -1.0, device="cuda")
    # one untimed call first: the first call on a device looks up the address of the built-in scratch
    call("pd_softmax_ce_fwd_static", _p(logits), dt, _p(target), rows, C, smoothing, padding_idx, scale, _p(lse_b),
         _p(loss_b), s)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before, _ = torch.cuda.mem_get_info()      # cudaMemGetInfo: also sees a cudaMalloc made inside the library
    call("pd_softmax_ce_fwd_static", _p(logits), dt, _p(target), rows, C, smoothing, padding_idx, scale, _p(lse_b),
         _p(loss_b), s)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert torch.cuda.memory_allocated() == before
    assert free_after >= free_before, "the entry point took %d bytes of device memory" % (free_before - free_after)
    return (loss_a.item(), lse_a), (loss_b.item(), lse_b)


def test_static_scratch_variant_matches_caller_scratch_variant():
    g = torch.Generator().manual_seed(77)
    # first call: many rows; second call: fewer rows and other values, so stale scratch from the
    # first call would show up if the kernel read anything it did not write
    cases = [(4096, 1000, torch.float32, 0.0, -1), (37, 32320, torch.bfloat16, 0.1, 0)]
    for rows, C, dtype, smoothing, pad in cases:
        logits = (torch.randn(rows, C, generator=g) * 3).to("cuda").to(dtype)
        target = torch.randint(0, C, (rows,), generator=g).to("cuda")
        if pad >= 0:
            target[::3] = pad
        (la, lse_a), (lb, lse_b) = _both(logits, target, smoothing, pad, 1.0 / 16)
        assert abs(la - lb) <= 1e-6 * max(1.0, abs(la)), (la, lb)
        assert torch.allclose(lse_a, lse_b, rtol=1e-6, atol=1e-6)


def test_static_scratch_variant_rejects_oversize():
    limit = _lib.load().pd_softmax_ce_static_max_rows()
    assert limit == 65536
    rows = limit + 1
    logits = torch.zeros(rows, 8, device="cuda")
    target = torch.zeros(rows, dtype=torch.int64, device="cuda")
    lse, loss = torch.empty(rows, device="cuda"), torch.empty((), device="cuda")
    with pytest.raises(_lib.PipedreamB200Error) as e:
        call("pd_softmax_ce_fwd_static", _p(logits), 0, _p(target), rows, 8, 0.0, -1, 1.0, _p(lse), _p(loss),
             ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert "exceed the built-in scratch" in str(e.value)
