"""tcgen05 grouped fp8 GEMM against a float32 PyTorch reference of the same op (operands
de-quantised, matmul in fp32, epilogue in fp32)."""

from __future__ import annotations

import pytest
import torch

from pplx_garden.ops import (
    MODE_BF16,
    MODE_SWIGLU_QUANT,
    dequantize_1x128,
    dequantize_128x128,
    grouped_fp8_gemm,
    quantize_1x128,
    quantize_128x128,
)

pytestmark = pytest.mark.gpu


def _layout(counts: list[int], padding: int) -> tuple[list[int], int]:
    starts, row = [], 0
    for n in counts:
        starts.append(row)
        row += -(-n // padding) * padding
    return starts, row


def _make(counts, K, N, padding, seed=0, unit_scales=False, pow2=False):
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device="cpu").manual_seed(seed)
    starts, rows = _layout(counts, padding)
    rows = max(rows, 1)
    E = len(counts)
    x = torch.randn((rows, K), generator=gen)
    w = torch.randn((E, N, K), generator=gen) * (K ** -0.5)
    if unit_scales:
        # values exactly representable in e4m3 with every scale equal to 2^-k: isolates the
        # tensor-core path (descriptors, swizzle, TMEM layout) from the scale handling
        x = torch.randint(-4, 5, (rows, K), generator=gen).float()
        w = torch.randint(-4, 5, (E, N, K), generator=gen).float() * 0.125
        x[:, ::128] = 448.0 / 64      # pin every block's amax so that all scales are equal
        w[:, ::128, ::128] = 448.0 / 512
    aq, a_s = quantize_1x128(x, pow2=pow2)
    bq, b_s = quantize_128x128(w, pow2=pow2)
    return (aq.to(dev), a_s.to(dev), bq.to(dev), b_s.to(dev),
            torch.tensor(counts, dtype=torch.int32, device=dev), starts, rows)


@pytest.mark.parametrize("counts,K,N,padding,unit", [
    ([128], 128, 256, 1, True),
    ([128], 512, 256, 1, True),
    ([128], 512, 256, 1, False),
    ([200, 0, 37, 128], 1024, 512, 1, False),
    ([5, 300, 64], 2048, 768, 16, False),
    ([1024] * 4, 768, 2048, 1, False),
    ([(7 * i) % 40 for i in range(100)], 256, 256, 1, False),   # many small experts, several per lane of the scan
    ([3] * 128, 128, 256, 4, False),
])
@pytest.mark.parametrize("tile_rows", [128, 256])
@pytest.mark.parametrize("scales", ["fp32", "pow2"])
def test_bf16_epilogue(counts, K, N, padding, unit, tile_rows, scales) -> None:
    aq, a_s, bq, b_s, cnt, starts, rows = _make(counts, K, N, padding, unit_scales=unit, pow2=scales == "pow2")
    out = torch.full((rows, N), float("nan"), dtype=torch.bfloat16, device=aq.device)
    flag = torch.zeros(1, dtype=torch.int32, device=aq.device)
    grouped_fp8_gemm(aq, a_s, bq, b_s, cnt, out, mode=MODE_BF16, expert_padding=padding, error_flag=flag,
                     tile_rows=tile_rows, scale_format=scales)
    torch.cuda.synchronize()
    assert flag.item() == 0, f"kernel reported a wait that ran out (code {flag.item()})"
    a = dequantize_1x128(aq, a_s)
    b = dequantize_128x128(bq, b_s)
    for e, (start, n) in enumerate(zip(starts, counts)):
        if n == 0:
            continue
        want = a[start:start + n] @ b[e].T
        got = out[start:start + n].float()
        torch.testing.assert_close(got, want, rtol=2e-2, atol=2e-2 * want.abs().max().item() / 8 + 1e-3,
                                   msg=lambda m, e=e: f"expert {e}: {m}")


@pytest.mark.parametrize("counts,K,I,padding", [
    ([128], 256, 128, 1),
    ([90, 0, 260], 1024, 256, 1),
    ([64, 512, 3], 2048, 768, 8),
])
@pytest.mark.parametrize("tile_rows", [128, 256])
@pytest.mark.parametrize("scales", ["fp32", "pow2"])
def test_swiglu_quant_epilogue(counts, K, I, padding, tile_rows, scales) -> None:
    N = 2 * I
    pow2 = scales == "pow2"
    aq, a_s, bq, b_s, cnt, starts, rows = _make(counts, K, N, padding, seed=1, pow2=pow2)
    out = torch.zeros((rows, I), dtype=torch.uint8, device=aq.device).view(torch.float8_e4m3fn)
    out_s = torch.zeros((rows, I // 128), dtype=torch.float32, device=aq.device)
    flag = torch.zeros(1, dtype=torch.int32, device=aq.device)
    grouped_fp8_gemm(aq, a_s, bq, b_s, cnt, out, out_s, mode=MODE_SWIGLU_QUANT, expert_padding=padding,
                     error_flag=flag, tile_rows=tile_rows, scale_format=scales)
    torch.cuda.synchronize()
    assert flag.item() == 0
    a = dequantize_1x128(aq, a_s)
    b = dequantize_128x128(bq, b_s)
    for e, (start, n) in enumerate(zip(starts, counts)):
        if n == 0:
            continue
        d = a[start:start + n] @ b[e].T
        gate, up = d[:, :I], d[:, I:]
        want = torch.nn.functional.silu(gate) * up
        got = dequantize_1x128(out[start:start + n], out_s[start:start + n])
        # e4m3 keeps 3 mantissa bits: relative error up to 2^-4 of the block maximum (of twice the
        # block maximum when the scale was rounded up to a power of two)
        block_max = want.reshape(n, I // 128, 128).abs().amax(-1).repeat_interleave(128, dim=1)
        assert ((got - want).abs() <= (0.14 if pow2 else 0.07) * block_max + 1e-4).all(), f"expert {e}"
        want_scale = want.reshape(n, I // 128, 128).abs().amax(-1).clamp_min(1e-10) / 448.0
        if pow2:
            got_scale = out_s[start:start + n]
            assert (torch.frexp(got_scale)[0] == 0.5).all(), "scales must be powers of two"
            ratio = got_scale / want_scale
            assert ((ratio >= 0.98) & (ratio <= 2.04)).all(), f"expert {e}: scale is not the next power of two"
        else:
            torch.testing.assert_close(out_s[start:start + n], want_scale, rtol=2e-2, atol=1e-8)
