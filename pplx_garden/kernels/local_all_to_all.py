"""Several expert-parallel ranks played by ONE process on ONE GPU.

Each launch covers all ranks at once (the kernels take the rank from ``blockIdx.y``), and
every rank's "peer" buffers live on the same device. This exercises the complete multi-rank
protocol (count exchange, record placement, arrival flags, replication across dp groups)
where only one GPU is available, and lets a profiler look at the multi-rank kernels on a
single device. Separate processes or launches per rank on one GPU would not do: kernels
that wait for one another are not guaranteed to run concurrently.

The reference has no equivalent; it tests multi-rank behaviour only on multi-GPU machines
with NICs (tests/p2p_all_to_all/test_p2p_all_to_all.py:237-557).
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from pplx_garden.native.p2p_all_to_all import AllToAllContext
from pplx_garden.utils.math import ceil_div


class LocalAllToAllGroup:
    def __init__(
        self,
        *,
        world_size: int,
        dp_size: int = 1,
        max_num_tokens: int,
        num_experts: int,
        expert_padding: int,
        hidden_dim: int,
        hidden_dim_scale: Optional[int],
        in_dtype: torch.dtype,
        out_dtype: torch.dtype,
        scale_dtype: Optional[torch.dtype],
        num_experts_per_token: int,
        device: torch.device,
        combine_mode: str = "per_route",
        num_blocks: int = 0,
        wait_limit_ms: int = 0,
        wire: Optional[str] = None,
        pow2_scales: bool = False,
    ) -> None:
        device = torch.device(device)
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.world_size = world_size
        self.quantize_mode = 2 if pow2_scales else 1
        self.dp_size = dp_size
        self.device = device
        self.hidden_dim = hidden_dim
        self.hidden_dim_scale = hidden_dim_scale
        self.in_dtype = in_dtype
        self.out_dtype = out_dtype
        self.scale_dtype = scale_dtype
        self.topk = num_experts_per_token
        self.num_local_experts = ceil_div(num_experts, world_size)
        props = torch.cuda.get_device_properties(device)
        common = dict(
            hidden_dim=hidden_dim,
            hidden_dim_scale=hidden_dim_scale,
            in_elemsize=in_dtype.itemsize,
            out_elemsize=out_dtype.itemsize,
            scale_elemsize=scale_dtype.itemsize if scale_dtype else None,
            max_num_tokens=max_num_tokens,
            num_experts=num_experts,
            expert_padding=expert_padding,
            num_experts_per_token=num_experts_per_token,
            dp_size=dp_size,
            world_size=world_size,
            combine_mode=combine_mode,
            num_blocks=num_blocks,
        )
        self.layout = AllToAllContext.layout(num_sms=props.multi_processor_count,
                                             virtual_ranks=world_size, wire=wire, **common)
        common["wire"] = self.layout["wire"]
        self.max_recv_rows: int = self.layout["max_recv_rows"]
        # torch's caching allocator returns 512-byte aligned blocks, which satisfies the
        # 128-byte alignment the kernels ask of the symmetric regions.
        self._sync = [torch.zeros(self.layout["sync_bytes"], dtype=torch.uint8, device=device)
                      for _ in range(world_size)]
        # record headers carry an epoch tag: the receive regions must start zeroed
        self._recv = [torch.zeros(self.layout["recv_bytes"], dtype=torch.uint8, device=device)
                      for _ in range(world_size)]
        torch.cuda.synchronize(device)
        sync_ptrs = [t.data_ptr() for t in self._sync]
        recv_ptrs = [t.data_ptr() for t in self._recv]
        self.context = AllToAllContext.create(
            out_dtype=out_dtype,
            rank=list(range(world_size)),
            sync_ptrs=[sync_ptrs] * world_size,
            recv_ptrs=[recv_ptrs] * world_size,
            device=device.index,
            wait_limit_ms=wait_limit_ms,
            **common,
        )

    # Each argument is a sequence with one entry per rank.
    def dispatch(
        self,
        out_expert_num_tokens: Sequence[torch.Tensor],
        out_expert_x: Sequence[torch.Tensor],
        out_expert_x_scale: Optional[Sequence[torch.Tensor]],
        dp_x: Sequence[torch.Tensor],
        dp_x_scale: Optional[Sequence[torch.Tensor]],
        indices: Sequence[torch.Tensor],
        weights: Sequence[torch.Tensor],
        bound_m: Optional[Sequence[Optional[torch.Tensor]]] = None,
        do_send: bool = True,
        do_recv: bool = True,
        logits: Optional[Sequence[torch.Tensor]] = None,
        logits_bias: Optional[Sequence[Optional[torch.Tensor]]] = None,
    ) -> None:
        """With ``logits`` (one [tokens, experts] tensor per rank) the kernel routes: it fills
        ``indices`` and ``weights`` instead of reading them."""
        send = recv = None
        if do_send:
            send = []
            for r in range(self.world_size):
                x = dp_x[r]
                quantize = self.quantize_mode if x.dtype != self.in_dtype else 0
                xs = None if dp_x_scale is None else dp_x_scale[r]
                bm = None if bound_m is None or bound_m[r] is None else bound_m[r].data_ptr()
                send.append((
                    x.shape[0], x.data_ptr(), x.stride(0) * x.element_size(),
                    None if xs is None else xs.data_ptr(),
                    None if xs is None else xs.stride(1),
                    None if xs is None else xs.stride(0),
                    indices[r].data_ptr(), indices[r].stride(0),
                    weights[r].data_ptr(), weights[r].stride(0), bm, quantize,
                ) + (() if logits is None else (
                    logits[r].data_ptr(), logits[r].stride(0), logits[r].dtype == torch.bfloat16,
                    None if logits_bias is None or logits_bias[r] is None else logits_bias[r].data_ptr(),
                )))
        if do_recv:
            recv = []
            for r in range(self.world_size):
                ox = out_expert_x[r]
                os_ = None if out_expert_x_scale is None else out_expert_x_scale[r]
                recv.append((
                    out_expert_num_tokens[r].data_ptr(), ox.data_ptr(),
                    ox.stride(0) * ox.element_size(),
                    None if os_ is None else os_.data_ptr(),
                    None if os_ is None else os_.stride(1),
                    None if os_ is None else os_.stride(0),
                    ox.shape[0],
                ))
        self.context.dispatch_multi(send, recv, torch.cuda.current_stream().cuda_stream)

    def combine(
        self,
        out_tokens: Sequence[torch.Tensor],
        indices: Sequence[torch.Tensor],
        weights: Sequence[torch.Tensor],
        expert_y: Optional[Sequence[torch.Tensor]],
        bound_m: Optional[Sequence[Optional[torch.Tensor]]] = None,
        do_send: bool = True,
        do_recv: bool = True,
        accumulate: bool = False,
    ) -> None:
        send = recv = None
        if expert_y is None:
            assert do_recv and not do_send, "expert_y may only be omitted when another kernel did the send"
        if do_send:
            send = [(y.data_ptr(), y.stride(0) * y.element_size()) for y in expert_y]
        if do_recv:
            recv = []
            for r in range(self.world_size):
                bm = None if bound_m is None or bound_m[r] is None else bound_m[r].data_ptr()
                recv.append((
                    indices[r].shape[0], out_tokens[r].data_ptr(), out_tokens[r].stride(0),
                    indices[r].data_ptr(), indices[r].stride(0),
                    weights[r].data_ptr(), weights[r].stride(0), bm, accumulate,
                ))
        self.context.combine_multi(send, recv, self.out_dtype if expert_y is None else expert_y[0].dtype,
                                   torch.cuda.current_stream().cuda_stream)

    def combine_send_external(self, bulk: bool = False) -> list:
        """One scatter descriptor per emulated rank (see P2PAllToAll.combine_send_external): the
        caller runs ``grouped_fp8_gemm(..., mode=MODE_BF16_SCATTER, scatter=desc[r])`` for every rank,
        then ``combine(..., expert_y=None, do_send=False, do_recv=True)``. The GEMMs wait for nobody,
        so they may run one after the other on this GPU."""
        return [(*d, 1) if bulk else d for d in self.context.combine_send_external()]

    def barrier(self) -> None:
        self.context.barrier(torch.cuda.current_stream().cuda_stream)

    def check(self) -> None:
        if self.context.failed():
            self.context.check()

    def destroy(self) -> None:
        torch.cuda.synchronize(self.device)
        self.context.destroy()
