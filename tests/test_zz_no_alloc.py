"""The allocation-free triangle multiplication (``ubm_trimul_noalloc``), called through its exported
C symbol, must give what the buffer-taking path gives.

It serves callers that cannot allocate device memory when they call (the allocator is owned by someone
else or must not be disturbed, or there is no tensor library at all), so its intermediates sit in a
fixed array inside the library.  That array is shared by all calls and keeps old contents, hence the
check on two calls in a row with different inputs and directions.  This file sorts last on purpose: a run
that stops at the first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_N = 160


def _symbol():
    from uplifting_biomolecular_modeling_b200.ops import native
    handle = ctypes.CDLL(str(native.library_path()))
    fn = handle.ubm_trimul_noalloc
    fn.argtypes = [ctypes.c_void_p] * 12 + [ctypes.c_int] * 3 + [ctypes.c_void_p] * 2
    fn.restype = ctypes.c_int
    return fn


def _weights(g):
    from uplifting_biomolecular_modeling_b200.ops import pair
    c = 128
    r = lambda *s, sc=1.0: torch.randn(*s, device="cuda", generator=g) * sc  # noqa: E731
    return pair.TrimulPacked.pack(1.0 + 0.1 * r(c), 0.1 * r(c), r(2 * c, c, sc=c ** -0.5), r(2 * c, c, sc=c ** -0.5),
                                  1.0 + 0.1 * r(c), 0.1 * r(c), r(c, c, sc=c ** -0.5), r(c, c, sc=c ** -0.5))


def _call(fn, z, mask, w, out, outgoing, residual, status):
    p = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())  # noqa: E731
    return fn(p(z), p(mask), p(w.w_in), p(w.in_colsum), p(w.in_colbias), p(w.wo), p(w.wg), p(w.o_colsum),
              p(w.o_colbias), p(w.g_colsum), p(w.g_colbias), p(out), z.shape[0], 1 if outgoing else 0,
              1 if residual else 0, p(status), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_noalloc_matches_buffer_path_twice_in_a_row():
    from uplifting_biomolecular_modeling_b200.ops import native, pair
    fn = _symbol()
    g = torch.Generator(device="cuda").manual_seed(11)
    w = _weights(g)
    status = native.status_tensor("cuda")
    # first call on this device: the address look-up and the kernels' attribute set-up happen here, so the
    # free-memory comparison below watches a call that has nothing left to set up
    zw = torch.zeros(8, 8, 128, device="cuda", dtype=torch.bfloat16)
    assert _call(fn, zw, None, w, torch.empty_like(zw), True, True, status) == 0
    torch.cuda.synchronize()
    for N, outgoing, residual in ((160, True, True), (96, False, False)):
        z = (torch.randn(N, N, 128, device="cuda", generator=g) + 0.2).bfloat16()
        mask = (torch.rand(N, N, device="cuda", generator=g) > 0.1).float()
        ref = pair.trimul_fused(z, mask, w, outgoing=outgoing, residual=residual)
        out = torch.empty_like(z)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]
        rc = _call(fn, z, mask, w, out, outgoing, residual, status)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before        # nothing came from torch's allocator
        assert torch.cuda.mem_get_info()[0] == free_before    # ... and nothing from the driver's either
        native.raise_on_status("cuda", "trimul_noalloc")
        # the same three kernels on the same operand layout as the buffer-taking path: the same bits
        assert torch.equal(out, ref), (N, outgoing, (out.float() - ref.float()).abs().max().item())
        # the output may be the input tensor itself
        z2 = z.clone()
        assert _call(fn, z2, mask, w, z2, outgoing, residual, status) == 0
        torch.cuda.synchronize()
        assert torch.equal(z2, ref)


def test_noalloc_rejects_sizes_beyond_the_scratch_array():
    fn = _symbol()
    g = torch.Generator(device="cuda").manual_seed(12)
    w = _weights(g)
    N = MAX_N + 8
    z = torch.zeros(N, N, 128, device="cuda", dtype=torch.bfloat16)
    out = torch.full_like(z, 7.0)
    assert _call(fn, z, None, w, out, True, True, None) == -4
    zbad = torch.zeros(100, 100, 128, device="cuda", dtype=torch.bfloat16)      # not a multiple of 8
    assert _call(fn, zbad, None, w, torch.empty_like(zbad), True, True, None) == -1
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())                                           # a refused call touches nothing
