"""Top-k routing kernel against its PyTorch statement."""

import pytest
import torch

from pplx_garden.ops import topk_route, topk_route_reference


def test_reference_on_cpu():
    logits = torch.tensor([[0.0, 3.0, 1.0, 2.0]])
    idx, w = topk_route_reference(logits, 2)
    assert idx.view(torch.int32).tolist() == [[1, 3]]
    assert torch.allclose(w, torch.softmax(torch.tensor([[3.0, 2.0]]), dim=-1))
    idx, _ = topk_route_reference(logits, 2, bias=torch.tensor([10.0, 0.0, 0.0, 0.0]))
    assert idx.view(torch.int32).tolist() == [[0, 1]]


@pytest.mark.gpu
@pytest.mark.parametrize("tokens,experts,k,dtype,with_bias", [
    (128, 256, 8, torch.float32, False),
    (4096, 256, 8, torch.float32, True),
    (2048, 128, 8, torch.bfloat16, False),
    (77, 60, 6, torch.float32, True),
    (5, 1024, 32, torch.float32, False),
    (33, 8, 8, torch.float32, False),
    (1, 384, 1, torch.bfloat16, True),
])
def test_topk_route_matches_reference(tokens, experts, k, dtype, with_bias):
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device="cpu").manual_seed(tokens * 31 + experts)
    logits = torch.randn((tokens, experts), generator=gen).to(dtype).to(dev)
    bias = (torch.randn(experts, generator=gen) * 0.5).to(dev) if with_bias else None
    idx, w = topk_route(logits, k, bias)
    ref_idx, ref_w = topk_route_reference(logits, k, bias)
    torch.cuda.synchronize()
    got, want = idx.view(torch.int32).cpu(), ref_idx.view(torch.int32).cpu()
    if dtype == torch.bfloat16:
        # bf16 logits tie often; the chosen sets must then agree as sets of (logit) values
        x = logits.float().cpu() + (0 if bias is None else bias.cpu())
        assert torch.equal(torch.gather(x, 1, got.long()), torch.gather(x, 1, want.long()))
    else:
        assert torch.equal(got, want)
    assert torch.allclose(w.cpu(), ref_w.cpu(), rtol=1e-4, atol=1e-6)
    assert torch.allclose(w.sum(dim=-1).cpu(), torch.ones(tokens), atol=1e-5)


@pytest.mark.gpu
def test_ties_go_to_the_lower_index():
    dev = torch.device("cuda", 0)
    logits = torch.zeros((3, 64), device=dev)
    idx, w = topk_route(logits, 4)
    assert idx.view(torch.int32).cpu().tolist() == [[0, 1, 2, 3]] * 3
    assert torch.allclose(w.cpu(), torch.full((3, 4), 0.25))
