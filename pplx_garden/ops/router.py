"""Top-k routing on the GPU: the k experts with the largest router logit per token and the
softmax of the chosen logits (weights renormalised over the chosen k), in the layout that
dispatch and combine take. The reference leaves routing to its callers
(tests/p2p_all_to_all/data.py:9-108 draws indices directly)."""

from __future__ import annotations

from typing import Optional

import torch

from pplx_garden import _native


def topk_route_reference(logits: torch.Tensor, topk: int,
                         bias: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Plain PyTorch statement of the op (any device): the oracle of the kernel's tests."""
    x = logits.float()
    keys = x if bias is None else x + bias.float()
    idx = torch.topk(keys, topk, dim=-1).indices
    weights = torch.softmax(torch.gather(x, 1, idx), dim=-1)
    return idx.to(torch.int32).view(torch.uint32), weights


def topk_route(logits: torch.Tensor, topk: int, bias: Optional[torch.Tensor] = None,
               out_indices: Optional[torch.Tensor] = None,
               out_weights: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """logits [tokens, experts] fp32 or bf16 on a CUDA device; optional bias [experts] fp32 that
    shifts the choice but not the weights. Returns (indices uint32 [tokens, k], weights fp32
    [tokens, k]), sorted by decreasing logit; ties go to the lower expert index."""
    if not logits.is_cuda:
        raise RuntimeError("topk_route runs on a CUDA device; use topk_route_reference on the CPU")
    assert logits.dim() == 2 and logits.stride(1) == 1
    assert logits.dtype in (torch.float32, torch.bfloat16)
    tokens, experts = logits.shape
    if bias is not None:
        assert bias.shape == (experts,) and bias.dtype == torch.float32 and bias.is_contiguous()
    if out_indices is None:
        out_indices = torch.empty((tokens, topk), dtype=torch.int32, device=logits.device).view(torch.uint32)
    if out_weights is None:
        out_weights = torch.empty((tokens, topk), dtype=torch.float32, device=logits.device)
    assert out_indices.shape == (tokens, topk) and out_indices.dtype == torch.uint32 and out_indices.stride(1) == 1
    assert out_weights.shape == (tokens, topk) and out_weights.dtype == torch.float32 and out_weights.stride(1) == 1
    _native.topk_route(
        logits.data_ptr(), logits.stride(0), logits.dtype == torch.bfloat16,
        0 if bias is None else bias.data_ptr(), out_indices.data_ptr(), out_indices.stride(0),
        out_weights.data_ptr(), out_weights.stride(0), tokens, experts, topk,
        torch.cuda.current_stream().cuda_stream)
    return out_indices, out_weights
