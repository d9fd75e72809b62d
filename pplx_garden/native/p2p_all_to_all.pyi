from typing import Any, Sequence

import torch

class AllToAllContext:
    @staticmethod
    def layout(
        *,
        hidden_dim: int,
        hidden_dim_scale: int | None = None,
        in_elemsize: int,
        out_elemsize: int,
        scale_elemsize: int | None = None,
        max_num_tokens: int,
        num_experts: int,
        expert_padding: int = 1,
        num_experts_per_token: int,
        dp_size: int = 1,
        world_size: int,
        combine_mode: str | int | None = None,
        num_blocks: int = 0,
        num_sms: int = 148,
        virtual_ranks: int = 1,
        wire: str | int | None = None,
        node_mask: int = 0,
    ) -> dict[str, int]: ...
    @staticmethod
    def create(
        *,
        hidden_dim: int,
        hidden_dim_scale: int | None = None,
        in_elemsize: int,
        out_elemsize: int,
        out_dtype: torch.dtype,
        scale_elemsize: int | None = None,
        max_num_tokens: int,
        max_recv_tokens: int | None = None,
        max_private_tokens: int | None = None,
        num_experts: int,
        expert_padding: int = 1,
        num_experts_per_token: int,
        rank: int | Sequence[int],
        dp_size: int = 1,
        node_size: int | None = None,
        world_size: int,
        num_routed_ptr: int | None = None,
        num_routed_mr: Any = None,
        send_buffer_ptr: int | None = None,
        send_buffer_mr: Any = None,
        recv_buffer_ptr: int | None = None,
        recv_buffer_mr: Any = None,
        sync_ptrs: list[int] | list[list[int]],
        send_ptrs: list[int] | None = None,
        recv_ptrs: list[int] | list[list[int]],
        device: int,
        imm_base: int | None = None,
        ranks: Any = None,
        transfer_engine: Any = None,
        worker_cpu: int | None = None,
        combine_mode: str | int | None = None,
        num_blocks: int = 0,
        wait_limit_ms: int = 0,
        wire: str | int | None = None,
        node_mask: int = 0,
    ) -> AllToAllContext: ...
    def config(self) -> dict[str, int]: ...
    def dispatch_send(
        self,
        num_tokens: int,
        x_ptr: int,
        x_stride: int,
        x_scale_ptr: int | None,
        x_scale_stride_elem: int | None,
        x_scale_stride_token: int | None,
        indices_ptr: int,
        indices_stride: int,
        weights_ptr: int,
        weights_stride: int,
        bound_m_ptr: int | None,
        stream: int,
        quantize: int = 0,  # 0 no, 1 bf16 -> e4m3 with fp32 1x128 scales, 2 the same with power-of-two scales
        logits_ptr: int | None = None,
        logits_stride: int = 0,
        logits_bf16: bool = False,
        logits_bias_ptr: int | None = None,
    ) -> None: ...
    def dispatch_recv(
        self,
        out_num_tokens_ptr: int,
        out_x_ptr: int,
        out_x_stride: int,
        out_x_scale_ptr: int | None,
        out_x_scale_stride_elem: int | None,
        out_x_scale_stride_token: int | None,
        stream: int,
        out_rows: int = 0,
    ) -> None: ...
    def dispatch(self, *args: Any, **kwargs: Any) -> None: ...
    def combine_send(
        self,
        expert_x_ptr: int,
        expert_x_stride: int,
        stream: int,
        expert_y_dtype: torch.dtype | None = None,
    ) -> None: ...
    def combine_send_external(self) -> list[tuple]: ...
    def combine_recv(
        self,
        num_tokens: int,
        num_recv_tokens: int | None,
        expert_y_dtype: torch.dtype,
        out_tokens_ptr: int,
        out_tokens_stride: int,
        indices_ptr: int,
        indices_stride: int,
        weights_ptr: int,
        weights_stride: int,
        bound_m_ptr: int | None,
        accumulate: bool,
        stream: int,
    ) -> None: ...
    def combine(self, *args: Any, **kwargs: Any) -> None: ...
    def dispatch_multi(self, send: list[tuple] | None, recv: list[tuple] | None, stream: int) -> None: ...
    def combine_multi(
        self, send: list[tuple] | None, recv: list[tuple] | None, expert_y_dtype: torch.dtype, stream: int
    ) -> None: ...
    def barrier(self, stream: int) -> None: ...
    def enable_proxy(
        self,
        transfer_engine: Any,
        peers: list[tuple[int, Any, Any]],
        local_rank: int = 0,
        worker_cpu: int = -1,
    ) -> None: ...
    def proxy_counters(self, local_rank: int = 0) -> tuple[int, int]: ...
    def trace(self, local_rank: int = 0) -> list[int]: ...
    def failed(self) -> bool: ...
    def check(self) -> None: ...
    def status(self, local_rank: int = 0) -> tuple[int, int, int, int, str]: ...
    def stats(self, local_rank: int = 0) -> list[int]: ...
    def iterations(self, local_rank: int = 0) -> list[int]: ...
    def set_team(self, team: int) -> None: ...
    def destroy(self) -> None: ...
