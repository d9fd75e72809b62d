"""Grouped block-scaled fp8 GEMM (tcgen05 / TMEM kernel in csrc/ops/grouped_gemm.cu) and the
torch-side quantisation helpers that define its number format.

Format: activations e4m3 with one fp32 scale per row and 128 columns (1x128), weights e4m3
with one fp32 scale per 128x128 block; ``scale = max(amax, 1e-10) / 448``.

With ``pow2=True`` the scale is rounded up to the next power of two (what a UE8M0 scale can
express). ``grouped_fp8_gemm(..., scale_format="pow2")`` then lets the tensor cores apply the scales
(``tcgen05.mma.kind::mxf8f6f4.block_scale``, csrc/ops/grouped_gemm_mx.cu) instead of folding every
K block's partial sums in the epilogue, which is about twice as fast.
"""

from __future__ import annotations

from typing import Optional

import torch

from pplx_garden import _native

MODE_SWIGLU_QUANT = 0
MODE_BF16 = 1
MODE_BF16_SCATTER = 2

SCALES_FP32 = 0
SCALES_POW2 = 1
_SCALE_FORMATS = {"fp32": SCALES_FP32, "pow2": SCALES_POW2, "ue8m0": SCALES_POW2, SCALES_FP32: SCALES_FP32,
                  SCALES_POW2: SCALES_POW2}


def round_scale_pow2(scale: torch.Tensor) -> torch.Tensor:
    """The smallest power of two that is >= each (positive, normal) fp32 scale."""
    bits = scale.contiguous().view(torch.int32)
    return ((bits + 0x007FFFFF) & 0x7F800000).view(torch.float32)


def quantize_1x128(x: torch.Tensor, pow2: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """[rows, K] float -> (e4m3 [rows, K], fp32 scales [rows, K // 128])."""
    rows, k = x.shape
    blocks = x.to(torch.float32).reshape(rows, k // 128, 128)
    scale = blocks.abs().amax(dim=-1).clamp_min(1e-10) * (1.0 / 448.0)
    if pow2:
        scale = round_scale_pow2(scale)
    q = (blocks / scale.unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q.reshape(rows, k), scale


def quantize_128x128(w: torch.Tensor, pow2: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """[..., N, K] float -> (e4m3 same shape, fp32 scales [..., N // 128, K // 128])."""
    *lead, n, k = w.shape
    blocks = w.to(torch.float32).reshape(*lead, n // 128, 128, k // 128, 128)
    scale = blocks.abs().amax(dim=(-3, -1)).clamp_min(1e-10) * (1.0 / 448.0)
    if pow2:
        scale = round_scale_pow2(scale)
    q = (blocks / scale.unsqueeze(-1).unsqueeze(-3)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q.reshape(*lead, n, k), scale


def dequantize_1x128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return q.to(torch.float32) * scale.repeat_interleave(128, dim=-1)


def dequantize_128x128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return q.to(torch.float32) * scale.repeat_interleave(128, dim=-2).repeat_interleave(128, dim=-1)


def grouped_fp8_gemm(
    a: torch.Tensor,
    a_scale: torch.Tensor,
    b: torch.Tensor,
    b_scale: torch.Tensor,
    expert_num_tokens: torch.Tensor,
    out: Optional[torch.Tensor],
    out_scale: Optional[torch.Tensor] = None,
    *,
    mode: int,
    expert_padding: int = 1,
    error_flag: Optional[torch.Tensor] = None,
    num_ctas: int = 0,
    wait_cycles: Optional[torch.Tensor] = None,
    debug_skip: int = 0,
    trace: Optional[torch.Tensor] = None,
    scatter: Optional[tuple] = None,
    tile_rows: int = 0,
    scale_format: str | int = "fp32",
) -> None:
    """``out[rows of expert e] = epilogue(dequant(a rows) @ dequant(b[e]).T)``.

    a [rows, K] e4m3, a_scale [rows, K/128] fp32 (any strides), b [E, N, K] e4m3 contiguous,
    b_scale [E, N/128, K/128] fp32 contiguous, expert_num_tokens [E] int32 on the device
    (rows are expert-major, each expert's block starting at a multiple of ``expert_padding``).
    mode MODE_SWIGLU_QUANT: b = [gate; up], out [rows, N/2] e4m3 and out_scale [rows, N/256];
    mode MODE_BF16: out [rows, N] bf16.
    mode MODE_BF16_SCATTER: no ``out``; ``scatter`` is the descriptor from
    ``P2PAllToAll.combine_send_external()``: every bf16 row goes straight into the combine receive
    buffer of the GPU its token came from (peer stores), and the kernel signals the receivers.
    ``tile_rows``: 256 = pairs of CTAs per tile (each CTA loads half of B), 128 = one CTA per tile,
    better for experts with few rows; 0 picks by ``rows / experts`` (capacity, not the counts).
    ``scale_format``: "fp32" takes any scales; "pow2" (or "ue8m0") promises that every scale of
    ``a_scale`` and ``b_scale`` is a power of two (``quantize_*(..., pow2=True)``; a scale that is not
    is truncated to the one below) and runs the block-scaled MMA kernel, whose SwiGLU epilogue
    writes power-of-two scales as well. The profiling arguments below are for "fp32" only.
    ``wait_cycles`` (int64 [num CTAs, 4], optional) receives the cycles each pipeline role spent
    waiting: producer for a free stage, MMA for a free accumulator, MMA for operands, epilogue
    for partial sums. ``debug_skip`` (profiling only, wrong results) removes a stage: 1 the
    epilogue's reads, 2 the MMAs, 4 the TMA loads; 8 issues every MMA twice. ``trace`` (int64 [64, 8], optional) receives SM clock
    readings for the tiles of CTA 0: epilogue tile start / first partial sums / K loop done / stored,
    MMA first issue / last commit, producer first / last load.
    """
    assert a.dtype == torch.float8_e4m3fn and b.dtype == torch.float8_e4m3fn
    assert a.dim() == 2 and b.dim() == 3 and b.is_contiguous() and b_scale.is_contiguous()
    assert a.stride(1) == 1 and (out is None or out.stride(1) == 1)
    rows, k = a.shape
    e, n, kb = b.shape
    assert kb == k and a_scale.shape == (rows, k // 128) and b_scale.shape == (e, n // 128, k // 128)
    assert a_scale.dtype == torch.float32 and b_scale.dtype == torch.float32
    assert expert_num_tokens.dtype == torch.int32 and expert_num_tokens.shape == (e,)
    if mode == MODE_SWIGLU_QUANT:
        assert out.dtype == torch.float8_e4m3fn and out.shape == (rows, n // 2)
        assert out_scale is not None and out_scale.shape == (rows, n // 256) and out_scale.dtype == torch.float32
        assert out_scale.stride(1) == 1
    elif mode == MODE_BF16_SCATTER:
        assert out is None and scatter is not None
    else:
        assert out.dtype == torch.bfloat16 and out.shape == (rows, n)
    if _SCALE_FORMATS[scale_format] == SCALES_POW2 and (wait_cycles is not None or debug_skip != 0):
        raise ValueError("wait_cycles and debug_skip belong to the fp32-scale kernel; the pow2 kernel has trace= only")
    if error_flag is None:
        error_flag = torch.zeros(1, dtype=torch.int32, device=a.device)
    _native.grouped_fp8_gemm(
        a.data_ptr(), a.stride(0) * a.element_size(), a_scale.data_ptr(), a_scale.stride(0), a_scale.stride(1),
        b.data_ptr(), b_scale.data_ptr(), expert_num_tokens.data_ptr(), a.data_ptr() if out is None else out.data_ptr(),
        16 if out is None else out.stride(0) * out.element_size(), 0 if out_scale is None else out_scale.data_ptr(),
        0 if out_scale is None else out_scale.stride(0), error_flag.data_ptr(), e, n, k, expert_padding, rows, mode,
        num_ctas, torch.cuda.current_stream().cuda_stream,
        0 if wait_cycles is None else wait_cycles.data_ptr(), debug_skip,
        0 if trace is None else trace.data_ptr(), scatter, tile_rows, _SCALE_FORMATS[scale_format])
