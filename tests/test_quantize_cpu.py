"""The torch-side fp8 block quantisers (the number format of dispatch and of the expert GEMMs) on
CPU: scale definition, power-of-two rounding, round trip error."""

from __future__ import annotations

import torch

from pplx_garden.kernels import oracle
from pplx_garden.ops.grouped_gemm import (
    dequantize_128x128,
    dequantize_1x128,
    quantize_128x128,
    quantize_1x128,
    round_scale_pow2,
)


def _is_pow2(t: torch.Tensor) -> bool:
    return bool((torch.frexp(t)[0] == 0.5).all())


def test_round_scale_pow2_is_the_next_power_of_two() -> None:
    s = torch.tensor([1.0, 1.0000001, 0.75, 0.5, 3.1e-6, 448.0, 2.0 ** -20, 1e-10 / 448.0])
    r = round_scale_pow2(s)
    assert _is_pow2(r)
    assert (r >= s).all() and (r < 2 * s).all()
    assert r[0] == 1.0 and r[3] == 0.5 and r[1] == 2.0 and r[2] == 1.0


def test_quantize_1x128_scale_definition_and_round_trip() -> None:
    gen = torch.Generator().manual_seed(0)
    x = torch.randn((33, 512), generator=gen) * torch.logspace(-3, 3, 33).unsqueeze(1)
    for pow2 in (False, True):
        q, s = quantize_1x128(x, pow2=pow2)
        assert q.dtype == torch.float8_e4m3fn and s.shape == (33, 4)
        amax = x.reshape(33, 4, 128).abs().amax(-1)
        if pow2:
            assert _is_pow2(s)
            assert (s >= amax / 448.0 * (1 - 1e-6)).all() and (s < 2 * amax / 448.0 * (1 + 1e-6)).all()
        else:
            torch.testing.assert_close(s, amax / 448.0)
        back = dequantize_1x128(q, s)
        # e4m3 keeps three mantissa bits: the error stays within 1/14 of the largest representable value of the block
        bound = (s * 448.0 / 14.0).repeat_interleave(128, dim=1)
        assert ((back - x).abs() <= bound).all()
        # the oracle's quantiser (the reference for the quantisation fused into dispatch) agrees bit for bit
        oq, os_ = oracle.quantize_1x128(x, pow2=pow2)
        assert torch.equal(oq.view(torch.uint8), q.view(torch.uint8)) and torch.equal(os_, s)


def test_quantize_128x128_blocks() -> None:
    gen = torch.Generator().manual_seed(1)
    w = torch.randn((3, 256, 384), generator=gen) * 0.02
    for pow2 in (False, True):
        q, s = quantize_128x128(w, pow2=pow2)
        assert s.shape == (3, 2, 3)
        if pow2:
            assert _is_pow2(s)
        back = dequantize_128x128(q, s)
        bound = (s * 448.0 / 14.0).repeat_interleave(128, dim=-2).repeat_interleave(128, dim=-1)
        assert ((back - w).abs() <= bound).all()
    # zero blocks do not divide by zero
    q, s = quantize_128x128(torch.zeros((1, 128, 128)), pow2=True)
    assert torch.isfinite(s).all() and (q.to(torch.float32) == 0).all()
