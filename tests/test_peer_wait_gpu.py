"""The bounded device-side wait of the stream barrier, on one GPU: a flag that nothing sets makes the wait run out
and the kernel reports it in the status word; with the flag set beforehand the same barrier passes."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_barrier_wait_runs_out_then_passes():
    from uplifting_biomolecular_modeling_b200.ops import native
    from uplifting_biomolecular_modeling_b200.parallel import symm
    dev = torch.device("cuda", 0)
    native.read_status(dev)                                   # start from a clean status word
    # two "ranks" whose flag arrays both live on this GPU: rank 0 waits for flags0[1] to reach the epoch
    flags0 = torch.zeros(64, dtype=torch.int32, device=dev)
    flags1 = torch.zeros(64, dtype=torch.int32, device=dev)
    ptrs = symm.ptr_array([flags0.data_ptr(), flags1.data_ptr()])
    st = native.status_tensor(dev)
    stream = native.current_stream(dev)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = native.lib().ubm_peer_barrier(ptrs, 0, 2, 1, 50, native.ptr(st), stream)        # limit 50 ms
    t1.record()
    assert rc == 0
    torch.cuda.synchronize()
    assert 30.0 < t0.elapsed_time(t1) < 1000.0               # the kernel gave up after its limit, not at once, not late
    code, where, block, aux = native.read_status(dev)
    assert (code, where, aux) == (2, 90, 1), (code, where, aux)       # peer wait ran out, barrier site, waiting for rank 1
    assert int(flags1[0]) == 1                                # rank 0 had announced itself to its peer
    with pytest.raises(native.KernelFault):
        native.lib().ubm_peer_barrier(ptrs, 0, 2, 2, 50, native.ptr(st), stream)
        native.raise_on_status(dev, "barrier")
    # the peer's arrival written first (stream order): the same barrier passes and leaves the status clean
    rc = native.lib().ubm_set_flag(flags0.data_ptr(), 1, 3, stream)
    assert rc == 0
    rc = native.lib().ubm_peer_barrier(ptrs, 0, 2, 3, 50, native.ptr(st), stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert native.read_status(dev)[0] == 0
