"""Host side of the causal-attention op: which calls the kernel takes, which views it can describe with one tensor
map, and the fp32 statement that the GPU test compares against."""
import torch
import torch.nn.functional as F

from uplifting_biomolecular_modeling_b200.ops import causal


def test_supported_names_the_reason():
    q = torch.zeros(1, 8, 2, 128, dtype=torch.bfloat16)
    assert causal.supported(q, q, q) == "not_cuda"
    assert causal.ENABLED in (True, False)


def test_row_views_that_one_tensor_map_can_describe():
    qkv = torch.zeros(2, 16, 3, 4, 128, dtype=torch.bfloat16)
    q, k, v = qkv.unbind(2)
    assert causal._rows(q) is q and causal._rows(v) is v            # column slices of one projection output
    assert causal._rows(q.transpose(1, 2).contiguous().transpose(1, 2)).is_contiguous()   # head-major storage: copied
    odd = torch.zeros(1, 16, 4, 136, dtype=torch.bfloat16)[..., :128]
    assert causal._rows(odd).is_contiguous() and causal._rows(odd).stride(2) == 128


def test_reference_statement_matches_the_library_on_cpu():
    torch.manual_seed(0)
    q, k, v = torch.randn(2, 40, 4, 128), torch.randn(2, 40, 2, 128), torch.randn(2, 40, 2, 128)
    kk, vv = k.repeat_interleave(2, 2), v.repeat_interleave(2, 2)
    want = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2),
                                          is_causal=True).transpose(1, 2)
    assert torch.allclose(causal.reference(q, k, v), want, atol=1e-5)
    tail = causal.reference(q[:, -9:], k, v)                        # queries that are the last positions of the keys
    assert torch.allclose(tail, want[:, -9:], atol=1e-5)
