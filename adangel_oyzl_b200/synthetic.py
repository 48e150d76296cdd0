"""Seeded synthetic inputs with the canonical value distributions.

Stand-in for the reference's prepared Llama-2-7B traces (``python/adangel/trace/prepare.py:82-140``),
which need a model and a dataset that are not available offline: activations ~ N(0,1) with 0.5 % of
the K channels scaled x20 (outliers), weights ~ N(0, 0.02); activations are quantized per row to
INT8 (``quantization/int8.py:6-17``) and weights to MXFP4 with one UE8M0 scale per K32 block
(``quantization/mxfp4.py:147-180``, exact floor(log2) exponent).

The float draws always use torch's CPU generator, so a seed means the same bits everywhere; the
quantization runs with plain torch ops on whichever device is requested.
"""

from __future__ import annotations

from .schema import PreparedInputs

CANONICAL_SEED = 20250805  # configs/experiment/o0_o1_o2_4096.yaml:3 of the reference


def quantize_int8_per_row(x):
    import torch

    x32 = x.to(torch.float32)
    amax = x32.abs().amax(dim=1)
    scale = torch.where(amax == 0, torch.ones_like(amax), amax / 127.0)
    q = torch.round(x32 / scale[:, None]).clamp(-127, 127).to(torch.int8)
    return q.contiguous(), scale.contiguous()


def quantize_mxfp4(x, row_chunk: int = 2048):
    """Packed E2M1 codes [rows, K/2] and UE8M0 scale codes [rows, K/32] of a float matrix."""
    import torch

    rows, cols = x.shape
    if cols % 32:
        raise ValueError("K must be divisible by 32")
    packed = torch.empty((rows, cols // 2), dtype=torch.uint8, device=x.device)
    scales = torch.empty((rows, cols // 32), dtype=torch.uint8, device=x.device)
    for r0 in range(0, rows, row_chunk):
        blocks = x[r0:r0 + row_chunk].to(torch.float32).reshape(-1, cols // 32, 32)
        amax = blocks.abs().amax(dim=-1)
        _, e = torch.frexp(torch.where(amax == 0, torch.ones_like(amax), amax))
        exps = torch.where(amax == 0, torch.zeros_like(e), e - 3).clamp(-127, 127)
        scales[r0:r0 + row_chunk] = (exps + 127).to(torch.uint8)
        mag = torch.ldexp(blocks, -exps.unsqueeze(-1)).abs()
        code = ((mag > 0.25).to(torch.uint8) + (mag >= 0.75) + (mag > 1.25) + (mag >= 1.75)
                + (mag > 2.5) + (mag >= 3.5) + (mag > 5.0)).to(torch.uint8)
        code = code | ((blocks < 0).to(torch.uint8) << 3)
        code = code.reshape(-1, cols)
        packed[r0:r0 + row_chunk] = code[:, 0::2] | (code[:, 1::2] << 4)
    return packed, scales


def canonical_floats(m: int, n: int, k: int, seed: int = CANONICAL_SEED):
    import torch

    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g, dtype=torch.float32)
    idx = torch.randperm(k, generator=g)[: max(1, round(0.005 * k))]
    a[:, idx] *= 20.0
    w = torch.randn(n, k, generator=g, dtype=torch.float32) * 0.02
    return a, w


def canonical_inputs(m: int, n: int, k: int, seed: int = CANONICAL_SEED, device="cpu", sample_id=None) -> PreparedInputs:
    a, w = canonical_floats(m, n, k, seed)
    a, w = a.to(device), w.to(device)
    if a.is_cuda:
        # the CUDA quantizers (bit-identical to the torch functions above, without their temporaries)
        from . import kernels

        a_int8, a_scale = kernels.quantize_int8_per_row(a, check_finite=False)
        w_mxfp4, w_scale = kernels.quantize_mxfp4(w, check_finite=False)
    else:
        a_int8, a_scale = quantize_int8_per_row(a)
        w_mxfp4, w_scale = quantize_mxfp4(w)
    return PreparedInputs(sample_id or f"synthetic_{m}x{n}x{k}_seed{seed}", a_int8, a_scale, w_mxfp4, w_scale)
