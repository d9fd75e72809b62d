"""Expert-parallel dispatch / combine over NVLink peer memory.

``P2PAllToAll`` keeps the constructor and the ``dispatch`` / ``combine`` / ``destroy``
signatures of the reference's python/pplx_garden/kernels/p2p_all_to_all.py:50-534, so
serving code written against it runs unchanged. What happens underneath differs:

* every rank allocates two CUDA-VMM regions (flags + counts, and the receive buffers),
  exports them as POSIX file descriptors and maps every peer's regions, as the reference
  does for its NVLink path (`:205-261`); there is no send buffer, no RDMA registration
  and no host proxy thread, because the kernels push counts, tokens and arrival signals
  directly into the peers' memory;
* receive regions are sized for the worst case (each source token reaches a rank at most
  once), so ``max_private_tokens`` has nothing left to tune and is accepted for
  compatibility only; ``nets_per_gpu`` likewise;
* ranks outside ``node_group`` (another node, or the other half of this box when a test
  slices it into "nodes") are served by a host proxy thread that forwards what the kernels
  staged for them through a ``TransferEngine`` and writes their arrival flags after the data
  (csrc/a2a/a2a_proxy.h); on this build the engine's provider is the intra-box one.

Extensions (keyword-only, all optional): ``combine_mode="pre_reduce"`` makes the expert
ranks apply the routing weights given at dispatch time and send one partial sum per
(token, expert rank) instead of one row per route; passing bf16 ``dp_x`` to a context
whose ``in_dtype`` is ``float8_e4m3fn`` with ``hidden_dim_scale = hidden_dim // 128`` and
``dp_x_scale=None`` quantises on the fly (one fp32 scale per 1x128 block; with
``pow2_scales=True`` every scale is rounded up to a power of two, which the block-scaled expert
GEMM, ``grouped_fp8_gemm(scale_format="pow2")``, needs); ``wire`` picks
the format on the wire: ``"ll"`` (128-byte lines that carry their own arrival flag, no fences,
one eighth more bytes: best for decode-sized calls), ``"plain"`` (contiguous records announced
by release stores: best for prefill-sized calls) or ``None`` (``"ll"`` up to 512 tokens per
call, the environment variable ``PPLX_A2A_WIRE`` overrides).
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

from pplx_garden.distributed import ParallelGroup
from pplx_garden.kernels.all_to_all import AllToAllKernel
from pplx_garden.native.cumem import (
    CUMemAllocHandle,
    CUMemExportHandle,
    CUMemHandleKind,
    CUMemMapping,
)
from pplx_garden.native.p2p_all_to_all import AllToAllContext
from pplx_garden.utils import logging_utils
from pplx_garden.utils.math import ceil_div

logger = logging_utils.get_logger(__name__)

_NVLINK_DOMAIN = 8


@dataclass
class _RankRegions:
    sync_handle: CUMemExportHandle
    recv_handle: CUMemExportHandle


@dataclass
class _PeerMappings:
    sync: CUMemMapping
    recv: CUMemMapping


def _sig(t: Optional[torch.Tensor]):
    """What the argument checks of dispatch / combine depend on."""
    if t is None:
        return None
    return (t.data_ptr(), t.shape, t.stride(), t.dtype)


def check_layout_agreement(group: ParallelGroup, rank: int, layout: dict) -> None:
    """Collective over ``group``: raises ValueError on every rank that finds a peer whose layout
    (wire format, strides, offsets, sizes) differs from its own. Launch shape (``num_blocks``), the
    NVLink-domain mask and the wait limit may differ."""
    shape_keys = sorted(k for k in layout if k not in ("num_blocks", "node_mask", "wait_limit_ns"))
    mine = tuple((k, layout[k]) for k in shape_keys)
    for peer, theirs in enumerate(group.all_gather_object(mine)):
        if theirs != mine:
            diff = [k for (k, v), (_, w) in zip(mine, theirs) if v != w]
            raise ValueError(
                f"rank {rank} and rank {peer} disagree about the all-to-all layout ({', '.join(diff)}); "
                "check PPLX_A2A_WIRE and the constructor arguments on every rank")


class P2PAllToAll(AllToAllKernel):
    def __init__(
        self,
        *,
        max_num_tokens: int,
        num_experts: int,
        expert_padding: int,
        hidden_dim: int,
        hidden_dim_scale: Optional[int],
        in_dtype: torch.dtype,
        out_dtype: torch.dtype,
        scale_dtype: Optional[torch.dtype],
        num_experts_per_token: int,
        nets_per_gpu: int = 0,
        max_private_tokens: Optional[int] = None,
        device: torch.device,
        dp_group: Optional[ParallelGroup],
        node_group: Optional[ParallelGroup] = None,
        global_group: Optional[ParallelGroup],
        combine_mode: str = "per_route",
        num_blocks: int = 0,
        wait_limit_ms: int = 0,
        wire: Optional[str] = None,
        pow2_scales: bool = False,
    ) -> None:
        device = torch.device(device)
        if device.type != "cuda":
            raise ValueError("P2PAllToAll needs a CUDA device")
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        if (hidden_dim_scale is None) != (scale_dtype is None):
            raise ValueError("hidden_dim_scale and scale_dtype must be given together")
        if scale_dtype is not None and scale_dtype != torch.float32:
            raise ValueError("only float32 scales are supported")

        self._hidden_dim = hidden_dim
        # scales of the quantisation fused into dispatch are rounded up to powers of two
        # (for grouped_fp8_gemm(..., scale_format="pow2"))
        self._quantize_mode = 2 if pow2_scales else 1
        self._hidden_dim_scale = hidden_dim_scale
        self._num_experts_per_token = num_experts_per_token
        self._in_dtype = in_dtype
        self._out_dtype = out_dtype
        self._scale_dtype = scale_dtype
        self._device = device
        self._global_group = global_group
        self._dp_size = dp_group.size if dp_group is not None else 1

        rank = global_group.rank if global_group is not None else 0
        world_size = global_group.size if global_group is not None else 1
        # Ranks of `node_group` share an NVLink domain: their memory is mapped here and the kernels
        # write into it. Ranks outside it are served by a host proxy through a transfer engine, as
        # every inter-node rank is in the reference (p2p-all-to-all/src/a2a_worker.rs:340-455).
        # Unlike there, node_group=None means "all ranks are in one NVLink domain".
        node_ranks = list(range(world_size))
        if node_group is not None and node_group.size != world_size:
            node_ranks = sorted(node_group.all_gather_object(rank))
        if len(node_ranks) > _NVLINK_DOMAIN:
            raise NotImplementedError(
                f"an NVLink domain of {len(node_ranks)} ranks: at most {_NVLINK_DOMAIN} GPUs share a switch; "
                "pass node_group to name the ranks of this node")
        if world_size > 32:
            raise NotImplementedError("the rank masks of the kernels hold 32 ranks")
        self._node_ranks = node_ranks
        self._multi_node = len(node_ranks) != world_size
        node_mask = 0
        for r in node_ranks:
            node_mask |= 1 << r
        if self._multi_node:
            if wire not in (None, "plain"):
                raise ValueError("ranks outside the NVLink domain need wire='plain'")
            wire = "plain"
        self._rank = rank
        self._world_size = world_size
        self._num_local_experts = ceil_div(num_experts, world_size)
        self._max_num_tokens = max_num_tokens
        self._all_to_all: Optional[AllToAllContext] = None

        props = torch.cuda.get_device_properties(device)
        if self._multi_node and num_blocks == 0:
            # The engine's paged copies are kernels of their own: while a dispatch or combine
            # waits for rows that such a copy is to deliver, the copy must find a free SM.
            num_blocks = max(1, props.multi_processor_count - 16)
        layout = AllToAllContext.layout(
            hidden_dim=hidden_dim,
            hidden_dim_scale=hidden_dim_scale,
            in_elemsize=in_dtype.itemsize,
            out_elemsize=out_dtype.itemsize,
            scale_elemsize=scale_dtype.itemsize if scale_dtype else None,
            max_num_tokens=max_num_tokens,
            num_experts=num_experts,
            expert_padding=expert_padding,
            num_experts_per_token=num_experts_per_token,
            dp_size=self._dp_size,
            world_size=world_size,
            combine_mode=combine_mode,
            num_blocks=num_blocks,
            num_sms=props.multi_processor_count,
            wire=wire,
            node_mask=node_mask,
        )
        self._layout = layout
        self.max_recv_rows: int = layout["max_recv_rows"]
        # Every rank writes into its peers' buffers with its own idea of the layout: the wire format
        # (which an environment variable can override per process), strides and offsets must be
        # the same everywhere, or a receiver would wait for lines that never come.
        if global_group is not None and world_size > 1:
            check_layout_agreement(global_group, rank, layout)

        torch.cuda.set_device(device)
        handle_kind = CUMemHandleKind.FileDescriptor
        self._sync_handle = CUMemAllocHandle(layout["sync_bytes"], device, handle_kind)
        self._recv_handle = CUMemAllocHandle(layout["recv_bytes"], device, handle_kind)
        sync_mapping = self._sync_handle.map(device)
        recv_mapping = self._recv_handle.map(device)
        sync_mapping.to_tensor((sync_mapping.size,), torch.uint8).zero_()
        # record headers carry an epoch tag: the receive regions must start zeroed
        recv_mapping.to_tensor((recv_mapping.size,), torch.uint8).zero_()
        torch.cuda.synchronize(device)

        self._mappings: list[Optional[_PeerMappings]] = [None] * world_size
        self._mappings[rank] = _PeerMappings(sync_mapping, recv_mapping)
        sharing_group = node_group if self._multi_node else global_group
        if len(node_ranks) > 1:
            assert sharing_group is not None
            mine = (rank, _RankRegions(self._sync_handle.export(), self._recv_handle.export()))
            for peer, regions in sharing_group.all_gather_object(mine):
                if peer != rank:
                    self._mappings[peer] = _PeerMappings(
                        regions.sync_handle.bind(device).map(device),
                        regions.recv_handle.bind(device).map(device),
                    )
            # Every peer has imported our descriptors: the exporter may now close them.
            sharing_group.barrier()
            del mine

        # The transfer engine for the ranks outside the domain, and everybody's descriptors.
        self._engine = None
        proxy_peers = []
        if self._multi_node:
            from pplx_garden.fabric_lib import TransferEngine

            assert global_group is not None
            if os.environ.get("CUDA_MODULE_LOADING", "").upper() != "EAGER":
                logger.warning(
                    "ranks outside the NVLink domain are served by copies that this GPU executes itself "
                    "(intra-box provider): set CUDA_MODULE_LOADING=EAGER, or make sure no kernel is launched "
                    "for the first time while a dispatch or combine is in flight; lazy module loading holds "
                    "copies back until running kernels finish, and those kernels wait for the copies")
            self._engine = TransferEngine(max(nets_per_gpu, 1), [device.index])
            _, sync_desc = self._engine.register_memory(sync_mapping.data_ptr(), sync_mapping.size, device)
            _, recv_desc = self._engine.register_memory(recv_mapping.data_ptr(), recv_mapping.size, device)
            for peer, sd, rd in global_group.all_gather_object((rank, sync_desc, recv_desc)):
                if peer not in node_ranks:
                    proxy_peers.append((peer, sd, rd))

        self._all_to_all = AllToAllContext.create(
            hidden_dim=hidden_dim,
            hidden_dim_scale=hidden_dim_scale,
            in_elemsize=in_dtype.itemsize,
            out_elemsize=out_dtype.itemsize,
            out_dtype=out_dtype,
            scale_elemsize=scale_dtype.itemsize if scale_dtype else None,
            max_num_tokens=max_num_tokens,
            max_private_tokens=max_private_tokens,
            num_experts=num_experts,
            expert_padding=expert_padding,
            num_experts_per_token=num_experts_per_token,
            rank=rank,
            dp_size=self._dp_size,
            node_size=world_size,
            world_size=world_size,
            sync_ptrs=[0 if m is None else m.sync.data_ptr() for m in self._mappings],
            recv_ptrs=[0 if m is None else m.recv.data_ptr() for m in self._mappings],
            device=device.index,
            combine_mode=combine_mode,
            num_blocks=num_blocks,
            wait_limit_ms=wait_limit_ms,
            wire=layout["wire"],
            node_mask=node_mask,
        )
        if self._multi_node:
            cpus = []
            try:
                for group in type(self._engine).detect_topology():
                    if group.cuda_device == device.index:
                        cpus = group.cpus
            except Exception:
                cpus = []
            self._all_to_all.enable_proxy(self._engine, proxy_peers, 0, cpus[-1] if cpus else -1)
        self._validate_only = False
        self._num_experts = num_experts
        self._dispatch_args: dict = {}
        self._combine_args: dict = {}
        self._check_every = int(os.environ.get("PPLX_A2A_CHECK_EVERY", "0"))
        self._calls = 0

        # No rank may signal a peer whose flags are not zeroed yet.
        if global_group is not None:
            global_group.barrier()

    # ------------------------------------------------------------------
    @property
    def num_local_experts(self) -> int:
        return self._num_local_experts

    @property
    def context(self) -> AllToAllContext:
        assert self._all_to_all is not None
        return self._all_to_all

    def check(self) -> None:
        """Raise if a kernel of this context reported a failure (e.g. a wait that timed out).
        Cheap: reads a pinned host word, does not synchronise the stream."""
        assert self._all_to_all is not None
        if self._all_to_all.failed():
            self._all_to_all.check()

    # ------------------------------------------------------------------
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
        logits: Optional[torch.Tensor] = None,
        logits_bias: Optional[torch.Tensor] = None,
    ) -> None:
        """``logits`` ([tokens, num_experts] fp32 or bf16) fuses the routing into the dispatch: the
        kernel picks each token's top-k experts on ``logits + logits_bias``, takes the softmax over
        the chosen logits, WRITES them to ``indices`` / ``weights`` (pass these to ``combine``) and
        sends by them, all in the team that moves the token."""
        a2a = self._all_to_all
        assert a2a is not None
        assert do_send or do_recv
        if logits is not None:
            return self._dispatch_routed(out_expert_num_tokens, out_expert_x, out_expert_x_scale, dp_x,
                                         dp_x_scale, indices, weights, bound_m, do_send, do_recv, logits,
                                         logits_bias)
        # A serving loop calls with the same tensors step after step: the checks below run once
        # per distinct set of (address, shape, strides, dtype) and the packed arguments are kept.
        key = (_sig(out_expert_num_tokens), _sig(out_expert_x), _sig(out_expert_x_scale), _sig(dp_x),
               _sig(dp_x_scale), _sig(indices), _sig(weights), _sig(bound_m))
        cached = self._dispatch_args.get(key)
        if cached is not None:
            send, recv, out_rows, quantize = cached
            stream = torch.cuda.current_stream().cuda_stream
            if do_send and do_recv:
                a2a.dispatch(*send, *recv, stream, out_rows, quantize)
            elif do_send:
                a2a.dispatch_send(*send, stream, quantize)
            else:
                a2a.dispatch_recv(*recv, stream, out_rows)
            return
        num_tokens = dp_x.shape[0]
        K = self._num_experts_per_token
        H = self._hidden_dim

        assert out_expert_num_tokens.shape == (self._num_local_experts,)
        assert out_expert_num_tokens.dtype == torch.int32 and out_expert_num_tokens.stride(0) == 1
        assert out_expert_x.dim() == 2 and out_expert_x.shape[1] == H
        assert out_expert_x.stride(1) == 1 and out_expert_x.dtype == self._in_dtype
        out_rows = out_expert_x.shape[0]
        out_x_stride = out_expert_x.stride(0) * out_expert_x.element_size()

        if out_expert_x_scale is not None:
            assert out_expert_x_scale.dtype == self._scale_dtype
            out_scale = (out_expert_x_scale.data_ptr(), out_expert_x_scale.stride(1),
                         out_expert_x_scale.stride(0))
        else:
            out_scale = (None, None, None)

        assert dp_x.shape == (num_tokens, H) and dp_x.stride(1) == 1
        quantize = 0
        if dp_x.dtype != self._in_dtype:
            # fused quantisation: bf16 in, e4m3 + 1x128 fp32 scales on the wire
            assert dp_x.dtype == torch.bfloat16 and self._in_dtype == torch.float8_e4m3fn, (
                f"dp_x is {dp_x.dtype}, the context was built for {self._in_dtype}")
            assert dp_x_scale is None and self._hidden_dim_scale == H // 128
            assert out_expert_x_scale is not None
            quantize = self._quantize_mode
        if dp_x_scale is not None:
            assert self._scale_dtype is not None and self._hidden_dim_scale is not None
            assert out_expert_x_scale is not None
            assert dp_x_scale.dtype == self._scale_dtype
            in_scale = (dp_x_scale.data_ptr(), dp_x_scale.stride(1), dp_x_scale.stride(0))
        else:
            assert quantize or (self._scale_dtype is None and self._hidden_dim_scale is None)
            in_scale = (None, None, None)

        assert indices.shape == (num_tokens, K) and indices.stride(1) == 1
        assert indices.dtype == torch.uint32
        assert weights.shape == (num_tokens, K) and weights.stride(1) == 1
        assert weights.dtype == torch.float32
        if bound_m is not None:
            assert bound_m.numel() == 1 and bound_m.dtype == torch.int32
            bound_m_ptr = bound_m.data_ptr()
        else:
            bound_m_ptr = None

        stream = torch.cuda.current_stream().cuda_stream
        send = (num_tokens, dp_x.data_ptr(), dp_x.stride(0) * dp_x.element_size(), *in_scale,
                indices.data_ptr(), indices.stride(0), weights.data_ptr(), weights.stride(0),
                bound_m_ptr)
        recv = (out_expert_num_tokens.data_ptr(), out_expert_x.data_ptr(), out_x_stride, *out_scale)
        if len(self._dispatch_args) > 64:
            self._dispatch_args.clear()
        self._dispatch_args[key] = (send, recv, out_rows, quantize)
        if self._validate_only:
            return
        if do_send and do_recv:
            a2a.dispatch(*send, *recv, stream, out_rows, quantize)
        elif do_send:
            a2a.dispatch_send(*send, stream, quantize)
        else:
            a2a.dispatch_recv(*recv, stream, out_rows)

    def _dispatch_routed(self, out_expert_num_tokens, out_expert_x, out_expert_x_scale, dp_x, dp_x_scale,
                         indices, weights, bound_m, do_send, do_recv, logits, logits_bias) -> None:
        E = self._num_local_experts * self._world_size
        T = dp_x.shape[0]
        assert logits.dim() == 2 and logits.shape[0] == T and logits.shape[1] >= self._num_experts <= E
        assert logits.stride(1) == 1 and logits.dtype in (torch.float32, torch.bfloat16)
        if logits_bias is not None:
            assert logits_bias.dtype == torch.float32 and logits_bias.is_contiguous()
            assert logits_bias.numel() >= self._num_experts
        extra = dict(logits_ptr=logits.data_ptr(), logits_stride=logits.stride(0),
                     logits_bf16=logits.dtype == torch.bfloat16,
                     logits_bias_ptr=None if logits_bias is None else logits_bias.data_ptr())
        # the plain path validates everything else and caches the packed arguments
        key = (_sig(out_expert_num_tokens), _sig(out_expert_x), _sig(out_expert_x_scale), _sig(dp_x),
               _sig(dp_x_scale), _sig(indices), _sig(weights), _sig(bound_m))
        if key not in self._dispatch_args:
            self._validate_only = True
            try:
                self.dispatch(out_expert_num_tokens, out_expert_x, out_expert_x_scale, dp_x, dp_x_scale,
                              indices, weights, bound_m, do_send, do_recv)
            finally:
                self._validate_only = False
        send, recv, out_rows, quantize = self._dispatch_args[key]
        stream = torch.cuda.current_stream().cuda_stream
        a2a = self._all_to_all
        if do_send and do_recv:
            a2a.dispatch(*send, *recv, stream, out_rows, quantize, **extra)
        elif do_send:
            a2a.dispatch_send(*send, stream, quantize, **extra)
        else:
            a2a.dispatch_recv(*recv, stream, out_rows)

    # ------------------------------------------------------------------
    def combine(
        self,
        out_tokens: torch.Tensor,
        indices: torch.Tensor,
        weights: torch.Tensor,
        expert_y: Optional[torch.Tensor],
        bound_m: Optional[torch.Tensor] = None,
        do_send: bool = True,
        do_recv: bool = True,
        accumulate: bool = False,
    ) -> None:
        a2a = self._all_to_all
        assert a2a is not None
        assert do_send or do_recv
        assert not accumulate or self._dp_size == 1, "accumulate is not supported with dp_size > 1"
        key = (_sig(out_tokens), _sig(indices), _sig(weights), _sig(expert_y), _sig(bound_m), accumulate)
        cached = self._combine_args.get(key)
        if cached is not None and expert_y is not None:
            y_ptr, y_stride, num_tokens, y_dtype, y_rows, recv = cached
            stream = torch.cuda.current_stream().cuda_stream
            if do_send and do_recv:
                a2a.combine(y_ptr, y_stride, num_tokens, y_dtype, *recv, stream)
            elif do_send:
                a2a.combine_send(y_ptr, y_stride, stream, y_dtype)
            else:
                a2a.combine_recv(num_tokens, y_rows, y_dtype, *recv, stream)
            return
        K = self._num_experts_per_token
        H = self._hidden_dim
        num_tokens = indices.shape[0]

        assert out_tokens.shape == (num_tokens, H) and out_tokens.stride(1) == 1
        assert out_tokens.dtype == self._out_dtype
        assert indices.shape == (num_tokens, K) and indices.stride(1) == 1
        assert indices.dtype == torch.uint32
        assert weights.shape == (num_tokens, K) and weights.stride(1) == 1
        assert weights.dtype == torch.float32
        if expert_y is None:
            assert do_recv and not do_send, "expert_y may only be omitted when another kernel did the send"
        else:
            assert expert_y.dim() == 2 and expert_y.shape[1] == H and expert_y.stride(1) == 1
            assert expert_y.element_size() == self._out_dtype.itemsize, (
                "expert_y must have the element size of out_dtype")
        if bound_m is not None:
            assert bound_m.numel() == 1 and bound_m.dtype == torch.int32
            bound_m_ptr = bound_m.data_ptr()
        else:
            bound_m_ptr = None

        stream = torch.cuda.current_stream().cuda_stream
        if expert_y is None:
            recv = (out_tokens.data_ptr(), out_tokens.stride(0), indices.data_ptr(), indices.stride(0),
                    weights.data_ptr(), weights.stride(0), bound_m_ptr, accumulate, stream)
            a2a.combine_recv(num_tokens, 0, self._out_dtype, *recv)
            return
        y_ptr = expert_y.data_ptr()
        y_stride = expert_y.stride(0) * expert_y.element_size()
        recv = (out_tokens.data_ptr(), out_tokens.stride(0), indices.data_ptr(), indices.stride(0),
                weights.data_ptr(), weights.stride(0), bound_m_ptr, accumulate)
        if len(self._combine_args) > 64:
            self._combine_args.clear()
        self._combine_args[key] = (y_ptr, y_stride, num_tokens, expert_y.dtype, expert_y.shape[0], recv)
        if do_send and do_recv:
            a2a.combine(y_ptr, y_stride, num_tokens, expert_y.dtype, *recv, stream)
        elif do_send:
            a2a.combine_send(y_ptr, y_stride, stream, expert_y.dtype)
        else:
            a2a.combine_recv(num_tokens, expert_y.shape[0], expert_y.dtype, *recv, stream)

    # ------------------------------------------------------------------
    def barrier(self) -> None:
        """Device-side barrier of all ranks on the current stream: a one-block kernel that
        announces this rank on every peer and waits (bounded) for all of them. Collective.
        Cheaper and much tighter than an NCCL all-reduce for lining ranks up."""
        a2a = self._all_to_all
        assert a2a is not None
        a2a.barrier(torch.cuda.current_stream().cuda_stream)

    # ------------------------------------------------------------------
    def combine_send_external(self, bulk: bool = False) -> tuple:
        """Let another kernel play the combine's send phase. Returns the descriptor that
        ``pplx_garden.ops.grouped_fp8_gemm(..., mode=MODE_BF16_SCATTER, scatter=...)`` takes: the
        down projection then writes every row straight into the combine receive buffer of the
        GPU its token came from and signals the receivers when it is done. Counts as
        ``combine(do_send=True, do_recv=False)`` in the phase order; follow it with
        ``combine(..., expert_y=None, do_send=False, do_recv=True)``.
        Needs the per_route combine mode, dp_size 1 and a 2-byte out_dtype. The reference has no
        such path (its combine always reads ``expert_y`` back:
        p2p-all-to-all/a2a-kernels/src/a2a/a2a_combine_send.cu:20-235)."""
        a2a = self._all_to_all
        assert a2a is not None
        (desc,) = a2a.combine_send_external()
        # bulk: the GEMM hands row chunks to the bulk-copy engine instead of storing them itself
        return (*desc, 1) if bulk else desc

    # ------------------------------------------------------------------
    def destroy(self) -> None:
        """Tear down. Collective: every rank must call it."""
        if self._all_to_all is None:
            return
        torch.cuda.synchronize(self._device)
        # No peer may still be writing into our regions when they are unmapped.
        if self._global_group is not None:
            self._global_group.barrier()
        self._all_to_all.destroy()      # joins the proxy thread, if any
        self._all_to_all = None
        if self._engine is not None:
            self._engine.stop()
            self._engine = None
            if self._global_group is not None:
                self._global_group.barrier()   # no engine still has our regions mapped
        for m in self._mappings:
            if m is not None:
                m.sync.unmap()
                m.recv.unmap()
        self._mappings.clear()
        del self._sync_handle, self._recv_handle
        if self._global_group is not None:
            self._global_group.barrier()
