"""Dispatch / combine written with library collectives only: ``all_to_all_single`` for the
per-expert counts and for the payload, torch indexing for the permutations and the
weighted sum. This is the measured *baseline* the NVLink kernels are compared with (over
NCCL on GPUs); over Gloo it also runs on CPU-only machines, which is how the multi-process
logic of this package is tested without a GPU.

It implements the same ``AllToAllKernel`` protocol (dp_size 1 only); the split
send/recv phases are honoured by buffering, and every call synchronises with the host
once to learn the split sizes, as library all-to-alls require.
The reference names this path as its generic fallback
(python/pplx_garden/distributed/torch_group.py:232-240).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from pplx_garden.distributed.torch_group import TorchParallelGroup
from pplx_garden.kernels.all_to_all import AllToAllKernel
from pplx_garden.utils.math import ceil_div


class NcclAllToAll(AllToAllKernel):
    def __init__(self, *, max_num_tokens: int, num_experts: int, expert_padding: int,
                 hidden_dim: int, hidden_dim_scale: Optional[int], in_dtype: torch.dtype,
                 out_dtype: torch.dtype, scale_dtype: Optional[torch.dtype],
                 num_experts_per_token: int, device: torch.device,
                 global_group: Optional[TorchParallelGroup]) -> None:
        self._group = global_group
        self._pg = global_group.device_group if global_group is not None else None
        self._rank = global_group.rank if global_group is not None else 0
        self._world = global_group.size if global_group is not None else 1
        self._E = num_experts
        self._L = ceil_div(num_experts, self._world)
        self._K = num_experts_per_token
        self._H = hidden_dim
        self._pad = expert_padding
        self._in_dtype = in_dtype
        self._out_dtype = out_dtype
        self._device = torch.device(device)
        self._pending: Optional[dict] = None   # state between dispatch and combine
        self._recv_stash: Optional[dict] = None

    # -- helpers ---------------------------------------------------------
    def _a2a(self, out: torch.Tensor, inp: torch.Tensor, out_splits: list[int], in_splits: list[int]) -> None:
        if self._pg is None:
            out.copy_(inp)
            return
        if self._device.type == "cuda":
            dist.all_to_all_single(out, inp, out_splits, in_splits, group=self._pg)
            return
        # Gloo: emulate with an all-gather of padded chunks.
        width = inp.shape[1:]
        cap = torch.tensor([max(in_splits, default=0)], dtype=torch.int64)
        dist.all_reduce(cap, op=dist.ReduceOp.MAX, group=self._pg)
        cap_n = max(int(cap.item()), 1)
        padded = torch.zeros((self._world, cap_n, *width), dtype=torch.uint8 if inp.dtype == torch.float8_e4m3fn else inp.dtype)
        src = inp.view(torch.uint8) if inp.dtype == torch.float8_e4m3fn else inp
        off = 0
        for d, n in enumerate(in_splits):
            padded[d, :n] = src[off:off + n]
            off += n
        everything = torch.empty((self._world, *padded.shape), dtype=padded.dtype)
        dist.all_gather_into_tensor(everything.view(-1), padded.view(-1), group=self._pg)
        dst = out.view(torch.uint8) if out.dtype == torch.float8_e4m3fn else out
        off = 0
        for s, n in enumerate(out_splits):
            dst[off:off + n] = everything[s, self._rank, :n]
            off += n

    # -- dispatch --------------------------------------------------------
    def dispatch(self, out_expert_num_tokens, out_expert_x, out_expert_x_scale, dp_x, dp_x_scale,
                 indices, weights, bound_m=None, do_send=True, do_recv=True) -> None:
        if do_send:
            self._dispatch_send(dp_x, dp_x_scale, indices, bound_m)
        if do_recv:
            self._dispatch_recv(out_expert_num_tokens, out_expert_x, out_expert_x_scale)

    def _dispatch_send(self, dp_x, dp_x_scale, indices, bound_m) -> None:
        W, L, K = self._world, self._L, self._K
        T = dp_x.shape[0]
        if bound_m is not None:
            T = min(T, int(bound_m.item()))
        idx = indices[:T].to(torch.int64)
        flat_e = idx.reshape(-1)                       # [T*K] expert of each route
        order = torch.argsort(flat_e, stable=True)     # routes sorted by expert (=> by rank)
        src_tok = torch.div(order, K, rounding_mode="floor")
        send_x = dp_x[:T][src_tok].contiguous()
        send_scale = dp_x_scale[:T][src_tok].contiguous() if dp_x_scale is not None else None
        counts = torch.bincount(flat_e, minlength=W * L)[: W * L].reshape(W, L).to(torch.int64)
        recv_counts = torch.empty_like(counts)
        self._a2a(recv_counts, counts, [1] * W, [1] * W)   # recv_counts[s, le]: from rank s
        in_splits = counts.sum(dim=1).tolist()             # host sync
        out_splits = recv_counts.sum(dim=1).tolist()
        n_recv = sum(out_splits)
        recv_x = torch.empty((n_recv, self._H), dtype=dp_x.dtype, device=dp_x.device)
        self._a2a(recv_x, send_x, out_splits, in_splits)
        recv_scale = None
        if send_scale is not None:
            recv_scale = torch.empty((n_recv, send_scale.shape[1]), dtype=send_scale.dtype,
                                     device=send_scale.device)
            self._a2a(recv_scale, send_scale, out_splits, in_splits)
        self._recv_stash = dict(recv_x=recv_x, recv_scale=recv_scale, recv_counts=recv_counts,
                                out_splits=out_splits, in_splits=in_splits, order=order, T=T)

    def _dispatch_recv(self, out_expert_num_tokens, out_expert_x, out_expert_x_scale) -> None:
        st = self._recv_stash
        assert st is not None, "dispatch(do_recv=True) without a preceding send"
        W, L = self._world, self._L
        recv_counts = st["recv_counts"]                    # [W, L]
        totals = recv_counts.sum(dim=0)                    # [L]
        padded = torch.div(totals + self._pad - 1, self._pad, rounding_mode="floor") * self._pad
        starts = torch.cumsum(padded, 0) - padded          # [L]
        # received rows are ordered (source rank, local expert); their expert-major position:
        within = torch.cumsum(recv_counts, 0) - recv_counts   # [W, L] rows of earlier sources
        base = (starts.unsqueeze(0) + within).reshape(-1)      # [W*L]
        reps = recv_counts.reshape(-1)
        seg_start = torch.repeat_interleave(base, reps)
        seg_first = torch.repeat_interleave(torch.cumsum(reps, 0) - reps, reps)
        dest_rows = seg_start + (torch.arange(int(reps.sum()), device=reps.device) - seg_first)
        out_expert_x[dest_rows] = st["recv_x"]
        if out_expert_x_scale is not None and st["recv_scale"] is not None:
            out_expert_x_scale[dest_rows] = st["recv_scale"]
        out_expert_num_tokens.copy_(totals.to(torch.int32))
        self._pending = dict(dest_rows=dest_rows, out_splits=st["out_splits"],
                             in_splits=st["in_splits"], order=st["order"], T=st["T"])
        self._recv_stash = None

    # -- combine ---------------------------------------------------------
    def combine(self, out_tokens, indices, weights, expert_y, bound_m=None, do_send=True,
                do_recv=True, accumulate=False) -> None:
        st = self._pending
        assert st is not None, "combine without a preceding dispatch"
        if do_send:
            back = expert_y[st["dest_rows"]].contiguous()      # (source rank, expert) order
            ret = torch.empty((sum(st["in_splits"]), self._H), dtype=expert_y.dtype,
                              device=expert_y.device)
            self._a2a(ret, back, st["in_splits"], st["out_splits"])
            st["returned"] = ret
        if do_recv:
            ret = st["returned"]
            T, K = st["T"], self._K
            routes = torch.empty((T * K, self._H), dtype=torch.float32, device=ret.device)
            routes[st["order"]] = ret.to(torch.float32)      # back to (token, k) order
            w = weights[:T].to(torch.float32).unsqueeze(-1)
            acc = (routes.reshape(T, K, self._H) * w).sum(dim=1)
            if accumulate:
                acc = acc + out_tokens[:T].to(torch.float32)
            out_tokens[:T] = acc.to(out_tokens.dtype)
            self._pending = None

    def destroy(self) -> None:
        self._pending = None
        self._recv_stash = None
