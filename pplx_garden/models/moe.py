"""Expert-parallel MoE feed-forward layer, fused end to end on the GPU:

    route (softmax over the top-k logits) ->
    dispatch       bf16 tokens are quantised to e4m3 (1x128 scales) inside the kernel that
                   pushes them to the expert ranks over NVLink
    gate/up GEMM   grouped block-scaled fp8 GEMM on tcgen05 tensor cores with the SwiGLU and the
                   re-quantisation to e4m3 fused into its epilogue
    down GEMM      same kernel, bf16 epilogue
    combine        expert rows return to their home rank and are reduced with the routing weights

The reference provides only the dispatch and combine steps (with an identity expert in its
tests: tests/p2p_all_to_all/test_p2p_all_to_all.py:44-50); the expert computation and its
fusion with the communication are additions of this library.
"""

from __future__ import annotations

from typing import Optional

import torch

from pplx_garden.distributed import ParallelGroup
from pplx_garden.kernels.p2p_all_to_all import P2PAllToAll
from pplx_garden.ops import MODE_BF16, MODE_BF16_SCATTER, MODE_SWIGLU_QUANT, grouped_fp8_gemm, quantize_128x128
from pplx_garden.ops.router import topk_route, topk_route_reference
from pplx_garden.utils.math import ceil_div


def route_topk(logits: torch.Tensor, topk: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Top-k experts by logit and their softmax weights renormalised over the chosen k.
    Returns (indices uint32 [tokens, k], weights float32 [tokens, k])."""
    if logits.is_cuda:
        return topk_route(logits, topk)
    return topk_route_reference(logits, topk)


class ExpertParallelMoE:
    """Holds this rank's expert weights (fp8, 128x128 block scales) and the all-to-all context."""

    def __init__(
        self,
        *,
        hidden_dim: int,
        intermediate_dim: int,
        num_experts: int,
        num_experts_per_token: int,
        max_num_tokens: int,
        device: torch.device,
        global_group: Optional[ParallelGroup],
        w13: Optional[torch.Tensor] = None,   # [local experts, 2 * intermediate, hidden], any float dtype
        w2: Optional[torch.Tensor] = None,    # [local experts, hidden, intermediate]
        init_std: float = 0.02,
        seed: int = 0,
        combine_mode: str = "per_route",
        fused_combine: bool = False,
        fused_bulk: bool = False,
        scale_format: str = "pow2",
    ) -> None:
        assert hidden_dim % 256 == 0 and intermediate_dim % 128 == 0
        assert scale_format in ("pow2", "fp32")
        # "pow2": every scale (weights, dispatch's quantisation, the SwiGLU epilogue's) is a power of two
        # and the tensor cores apply them (block-scaled MMA); "fp32": any scale, folded in by the
        # GEMM's epilogue per K block, which is slower
        self.scale_format = scale_format
        pow2 = scale_format == "pow2"
        self.hidden_dim = hidden_dim
        self.intermediate_dim = intermediate_dim
        self.topk = num_experts_per_token
        self.device = torch.device(device)
        world = global_group.size if global_group is not None else 1
        rank = global_group.rank if global_group is not None else 0
        self.num_local_experts = ceil_div(num_experts, world)
        L = self.num_local_experts
        if w13 is None or w2 is None:
            gen = torch.Generator(device="cpu").manual_seed(seed + 1000 * rank)
            w13 = torch.randn((L, 2 * intermediate_dim, hidden_dim), generator=gen) * init_std
            w2 = torch.randn((L, hidden_dim, intermediate_dim), generator=gen) * init_std
        self.w13, self.w13_scale = (t.to(self.device) for t in quantize_128x128(w13, pow2=pow2))
        self.w2, self.w2_scale = (t.to(self.device) for t in quantize_128x128(w2, pow2=pow2))
        self.a2a = P2PAllToAll(
            max_num_tokens=max_num_tokens, num_experts=num_experts, expert_padding=1,
            hidden_dim=hidden_dim, hidden_dim_scale=hidden_dim // 128, in_dtype=torch.float8_e4m3fn,
            out_dtype=torch.bfloat16, scale_dtype=torch.float32,
            num_experts_per_token=num_experts_per_token, device=self.device, dp_group=None,
            node_group=None, global_group=global_group, combine_mode=combine_mode,
            # a down projection that sends its own rows writes them in the plain row format
            wire="plain" if fused_combine else None, pow2_scales=pow2)
        rows = self.a2a.max_recv_rows
        dev = self.device
        self.expert_num_tokens = torch.zeros(L, dtype=torch.int32, device=dev)
        self.expert_x = torch.zeros((rows, hidden_dim), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        self.expert_x_scale = torch.zeros((rows, hidden_dim // 128), dtype=torch.float32, device=dev)
        self.act = torch.zeros((rows, intermediate_dim), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        self.act_scale = torch.zeros((rows, intermediate_dim // 128), dtype=torch.float32, device=dev)
        self.expert_y = torch.zeros((rows, hidden_dim), dtype=torch.bfloat16, device=dev)
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=dev)
        # Tile shape of the expert GEMMs from the rows an expert can expect (the capacity of the
        # receive buffer is a worst case and would always say "large"): 256-row CTA-pair tiles for
        # big experts, 128-row single-CTA tiles otherwise. An expert's last tile is mostly padding
        # (the counts are ragged), and with fewer than about two 256-row tiles per expert that
        # costs the pairs more than their better operand reuse gains: 64 experts of 264 rows took
        # 163 us with pairs and 100 us with single CTAs (gate/up, hidden 2048).
        expected_rows = max_num_tokens * num_experts_per_token * world / max(num_experts, 1)
        self.tile_rows = 256 if expected_rows >= 512 else 128
        # fused_combine: the down projection writes its rows into the peers' combine buffers itself
        self.fused_combine = fused_combine
        self.fused_bulk = fused_bulk   # fused_combine through the bulk-copy engine
        assert not fused_combine or combine_mode == "per_route"

    def forward(self, x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor,
                out: Optional[torch.Tensor] = None, logits: Optional[torch.Tensor] = None,
                logits_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x bf16 [tokens, hidden]; indices uint32 and weights fp32 [tokens, k]. With ``logits``
        ([tokens, experts]) the routing is made inside the dispatch kernel, which fills ``indices``
        and ``weights``; without, they are inputs."""
        assert x.dtype == torch.bfloat16 and x.shape[1] == self.hidden_dim
        if out is None:
            out = torch.empty_like(x)
        self.a2a.dispatch(self.expert_num_tokens, self.expert_x, self.expert_x_scale, x, None, indices, weights,
                          logits=logits, logits_bias=logits_bias)
        self.gate_up()
        if self.fused_combine:
            self.down_and_send()
            self.a2a.combine(out, indices, weights, None, do_send=False, do_recv=True)
        else:
            self.down()
            self.a2a.combine(out, indices, weights, self.expert_y)
        return out

    def gate_up(self) -> None:
        """act = quantise(silu(x W_gate^T) * (x W_up^T)) on the rows dispatch delivered."""
        grouped_fp8_gemm(self.expert_x, self.expert_x_scale, self.w13, self.w13_scale, self.expert_num_tokens,
                         self.act, self.act_scale, mode=MODE_SWIGLU_QUANT, error_flag=self.error_flag,
                         tile_rows=self.tile_rows, scale_format=self.scale_format)

    def down_and_send(self) -> None:
        """The down projection and the combine's send phase in one kernel: every output row is
        written over NVLink into the combine receive buffer of the GPU its token came from. Always
        on 256-row tiles: their epilogue sends whole 128-byte lines, the single-CTA tiles' 64-byte
        halves (EP2, 64 experts of about 256 rows: 80.8 against 109.2 us)."""
        grouped_fp8_gemm(self.act, self.act_scale, self.w2, self.w2_scale, self.expert_num_tokens, None,
                         mode=MODE_BF16_SCATTER, error_flag=self.error_flag,
                         scatter=self.a2a.combine_send_external(self.fused_bulk),
                         tile_rows=256, scale_format=self.scale_format)

    def down(self) -> None:
        """expert_y = act W_down^T in bf16: the rows combine sends home."""
        grouped_fp8_gemm(self.act, self.act_scale, self.w2, self.w2_scale, self.expert_num_tokens,
                         self.expert_y, mode=MODE_BF16, error_flag=self.error_flag, tile_rows=self.tile_rows,
                         scale_format=self.scale_format)

    __call__ = forward

    def check(self) -> None:
        """Raise if any kernel of the layer reported a failed wait (synchronises)."""
        self.a2a.check()
        if int(self.error_flag.item()) != 0:
            raise RuntimeError(f"grouped GEMM gave up on a wait (code {int(self.error_flag.item())})")

    def destroy(self) -> None:
        self.a2a.destroy()
