"""tcgen05.mma with the A operand in tensor memory against a plain fp32 product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_ts_mma_matches_fp32():
    from uplifting_biomolecular_modeling_b200.ops import native
    from uplifting_biomolecular_modeling_b200.ops.native import c_void_p
    native.declare("ubm_tsmma_probe", [c_void_p] * 5)
    g = torch.Generator(device="cuda").manual_seed(21)
    a = torch.randn(128, 64, device="cuda", generator=g).bfloat16()
    b = torch.randn(64, 64, device="cuda", generator=g).bfloat16()
    d = torch.zeros(128, 64, device="cuda")
    st = native.status_tensor("cuda")
    rc = native.lib().ubm_tsmma_probe(native.ptr(a), native.ptr(b), native.ptr(d), native.ptr(st),
                                      native.current_stream("cuda"))
    assert rc == 0
    torch.cuda.synchronize()
    native.raise_on_status("cuda", "ts mma probe")
    ref = a.float() @ b.float().T
    assert (d - ref).abs().max().item() < 1e-2 * ref.abs().max().item()
