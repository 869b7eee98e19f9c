"""Host chunks, host-resident pair tensors, the LayerNorm guard, the resident item loop, the backend pin."""
import threading

import pytest
import torch

from uplifting_biomolecular_modeling_b200.host import resident
from uplifting_biomolecular_modeling_b200.mem import primitives as P
from uplifting_biomolecular_modeling_b200.seq import backend


def test_host_chunks_are_powers_of_two_and_reused():
    hc = P.HostChunks(min_bytes=1024, pin=False)
    a = hc.lease(1500)
    assert a.numel() == 2048
    hc.release(a)
    b = hc.lease(1100)
    assert b.data_ptr() == a.data_ptr() and hc.allocated_bytes == 2048 and hc.leases == 2
    assert hc.lease(10).numel() == 1024
    v = hc.view(b, (4, 8), torch.float32)
    assert v.shape == (4, 8) and v.dtype == torch.float32


def test_host_pair_row_and_column_windows():
    z = torch.randn(12, 12, 8)
    hp = P.HostPair.from_tensor(z, P.HostChunks(pin=False))
    assert torch.equal(hp.rows(3, 7), z[3:7]) and torch.equal(hp.cols(2, 5), z[:, 2:5])
    hp.map_rows(lambda blk, i0, i1: blk * 2 + i0, rows=5)
    want = torch.cat([z[i0:i0 + 5] * 2 + i0 for i0 in range(0, 12, 5)])
    assert torch.equal(hp.host, want)
    hp.release()


def test_layernorm_guard_chunks_above_the_limit():
    x = torch.randn(50, 7, 16)
    w, b = torch.randn(16), torch.randn(16)
    ref = torch.nn.functional.layer_norm(x, (16,), w, b)
    g = P.LayerNormGuard(limit=1000)
    torch.testing.assert_close(g(x, w, b), ref)
    assert g.chunked_calls == 1
    assert P.LayerNormGuard()(x, w, b).equal(ref)


def test_resident_loop_prepares_ahead_writes_behind_and_survives_bad_items():
    written, errors = [], []
    main = threading.get_ident()
    seen_threads = set()

    def prepare(i):
        seen_threads.add(threading.get_ident())
        if i == 3:
            raise ValueError("unreadable input")
        return i * 10

    def forward(x):
        assert threading.get_ident() == main            # the device-owning thread
        if x == 50:
            raise RuntimeError("forward failed")
        return x + 1

    st = resident.run_resident(range(7), prepare, forward, written.append, workers=2, depth=2,
                               on_error=lambda item, e: errors.append((item, type(e).__name__)))
    assert sorted(written) == [(0, 1), (1, 11), (2, 21), (4, 41), (6, 61)]
    assert st.items == 5 and sorted(st.failed) == [3, 5] and main not in seen_threads
    assert sorted(errors) == [(3, "ValueError"), (5, "RuntimeError")]
    assert st.words()["failed"] == 2


def test_backend_pin_and_token_budget():
    q = torch.randn(1, 2, 5, 8)
    with backend.pinned_backend("math") as name:
        out = torch.nn.functional.scaled_dot_product_attention(q, q, q)
    assert name == "math" and out.shape == q.shape
    with pytest.raises(ValueError):
        with backend.pinned_backend("turbo"):
            pass
    n = backend.tokens_within(10 * 2 ** 30, d_model=1024, layers=12)
    assert n == int(10 * 2 ** 30 * 0.85) // (1024 * 2 * 7)
    assert backend.tokens_within(10 * 2 ** 30, 1024, 12, ceiling=4096) == 4096
