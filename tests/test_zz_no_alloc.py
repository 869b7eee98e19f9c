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
    for N, outgoing, residual in ((160, True, True), (96, False, False)):
        z = (torch.randn(N, N, 128, device="cuda", generator=g) + 0.2).bfloat16()
        mask = (torch.rand(N, N, device="cuda", generator=g) > 0.1).float()
        ref = pair.trimul_fused(z, mask, w, outgoing=outgoing, residual=residual)
        out = torch.empty_like(z)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = _call(fn, z, mask, w, out, outgoing, residual, status)
        assert rc == 0
        assert torch.cuda.memory_allocated() == before        # nothing came from torch's allocator either
        torch.cuda.synchronize()
        native.raise_on_status("cuda", "trimul_noalloc")
        err = (out.float() - ref.float()).abs().max().item()
        scale = ref.float().abs().max().item()
        assert err <= 2e-2 * max(scale, 1.0), (N, outgoing, err, scale)


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
