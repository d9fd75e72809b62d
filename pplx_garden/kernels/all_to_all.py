"""Interface of an expert-parallel all-to-all implementation.

``dispatch`` moves every token to the ranks that own its top-k experts and lays the
received tokens out expert-major; ``combine`` brings the expert outputs back and reduces
them with the routing weights. Both can be split into a *send* and a *recv* half so that
other work can be overlapped in between. Same protocol as the reference's
python/pplx_garden/kernels/all_to_all.py:6-33.
"""

from __future__ import annotations

from typing import Optional, Protocol

import torch


class AllToAllKernel(Protocol):
    def dispatch(
        self,
        out_expert_num_tokens: torch.Tensor,
        out_expert_x: torch.Tensor,
        out_expert_x_scale: Optional[torch.Tensor],
        dp_x: torch.Tensor,
        dp_x_scale: Optional[torch.Tensor],
        indices: torch.Tensor,
        weights: torch.Tensor,
        bound_m: Optional[torch.Tensor] = None,
        do_send: bool = True,
        do_recv: bool = True,
    ) -> None: ...

    def combine(
        self,
        out_tokens: torch.Tensor,
        indices: torch.Tensor,
        weights: torch.Tensor,
        expert_y: torch.Tensor,
        bound_m: Optional[torch.Tensor] = None,
        do_send: bool = True,
        do_recv: bool = True,
        accumulate: bool = False,
    ) -> None: ...

    def destroy(self) -> None: ...
