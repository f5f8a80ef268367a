"""Number formats of the checkpoint and of the quantised execution paths (CPU reference codecs).

* E8M0 scale byte b -> 2^(b - 127) (b = 0 is the smallest scale 2^-127, 0xff is NaN);
* E4M3FN: max 448, NaN = 0x7f / 0xff, no infinities;
* E2M1 (FP4): magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6}, sign in bit 3, two values per byte with the
  LOW nibble first;
* activation quantisation: one scale per 1x128 block, amax floored at 1e-4, power-of-two scale
  2^ceil(log2(amax / 448));
* weight formats: FP8 with one E8M0 scale per 128x128 block; MXFP4 with one E8M0 scale per 32
  elements of a row;
* the QAT simulators (quantise -> dequantise with a bf16 write-back) and the orthonormal
  fast Walsh-Hadamard transform used in front of FP4 quantisation.

Counterpart of crates/ferrule-model/src/checkpoint/encoding.rs:14-300 and of the device decoders
in crates/ferrule-backend/native/cuda/implementations/portable/entrypoints.cu:63-66, :342-448.
"""
from __future__ import annotations

from typing import Tuple

import torch

E4M3_MAX = 448.0
FP4_MAX = 6.0
_FP4_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


# ---------------------------------------------------------------------------------------- E8M0
def e8m0_decode(b: torch.Tensor) -> torch.Tensor:
    """uint8 -> float32 scale 2^(b-127); 0xff -> NaN."""
    bi = b.to(torch.int32)
    out = torch.ldexp(torch.ones_like(bi, dtype=torch.float32), bi - 127)
    return torch.where(bi == 255, torch.full_like(out, float("nan")), out)


def e8m0_encode_ceil(scale: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= scale, as an E8M0 byte (clamped to [0, 254])."""
    e = torch.ceil(torch.log2(scale.float().clamp_min(2.0 ** -127)))
    return (e + 127).clamp(0, 254).to(torch.uint8)


# ---------------------------------------------------------------------------------------- E4M3
def e4m3_decode(b: torch.Tensor) -> torch.Tensor:
    """uint8 bit patterns -> float32."""
    return b.contiguous().view(torch.float8_e4m3fn).float()


def e4m3_encode(x: torch.Tensor) -> torch.Tensor:
    """float -> uint8 bit patterns, round-to-nearest-even, saturating at +-448."""
    return x.float().clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)


# ---------------------------------------------------------------------------------------- E2M1
def fp4_decode_nibbles(n: torch.Tensor) -> torch.Tensor:
    """4-bit codes (uint8 0..15) -> float32."""
    mag = _FP4_VALUES.to(n.device)[(n & 7).long()]
    return torch.where((n & 8) != 0, -mag, mag)


def fp4_encode_nibbles(x: torch.Tensor) -> torch.Tensor:
    """float -> 4-bit code of the nearest representable value (ties to the even code)."""
    xf = x.float()
    a = xf.abs().clamp(max=FP4_MAX)
    vals = _FP4_VALUES.to(x.device)
    d = (a.unsqueeze(-1) - vals).abs()
    # nearest; on a tie prefer the code with an even mantissa bit (codes 0,2,4,6)
    tie_break = torch.tensor([0.0, 1e-7, 0.0, 1e-7, 0.0, 1e-7, 0.0, 1e-7], device=x.device)
    code = (d + tie_break).argmin(-1).to(torch.uint8)
    return torch.where(xf < 0, code | 8, code)


def fp4_unpack(packed: torch.Tensor) -> torch.Tensor:
    """[..., n/2] bytes -> [..., n] float32 (low nibble = even element)."""
    lo, hi = packed & 0x0F, (packed >> 4) & 0x0F
    return torch.stack((fp4_decode_nibbles(lo), fp4_decode_nibbles(hi)), dim=-1).flatten(-2)


def fp4_pack(x: torch.Tensor) -> torch.Tensor:
    """[..., n] float -> [..., n/2] bytes (low nibble first)."""
    codes = fp4_encode_nibbles(x)
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).to(torch.uint8)


# ---------------------------------------------------------------------------------------- activations
def act_quant_fp8(x: torch.Tensor, block: int = 128, amax_floor: float = 1e-4) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row 1 x `block` dynamic quantisation -> (uint8 e4m3 codes [.., n], uint8 e8m0 scales [.., n/block])."""
    *lead, n = x.shape
    assert n % block == 0
    xb = x.float().reshape(*lead, n // block, block)
    amax = xb.abs().amax(-1).clamp_min(amax_floor)
    sb = e8m0_encode_ceil(amax / E4M3_MAX)
    q = e4m3_encode(xb / e8m0_decode(sb).unsqueeze(-1))
    return q.reshape(*lead, n), sb


def act_dequant_fp8(q: torch.Tensor, sb: torch.Tensor, block: int = 128) -> torch.Tensor:
    *lead, n = q.shape
    v = e4m3_decode(q).reshape(*lead, n // block, block)
    return (v * e8m0_decode(sb).unsqueeze(-1)).reshape(*lead, n)


# ---------------------------------------------------------------------------------------- weights
def weight_quant_fp8_block(w: torch.Tensor, block: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """[out, in] -> (uint8 codes [out, in], uint8 e8m0 scales [ceil(out/b), ceil(in/b)])."""
    o, i = w.shape
    ob, ib = (o + block - 1) // block, (i + block - 1) // block
    wp = torch.zeros(ob * block, ib * block, dtype=torch.float32, device=w.device)
    wp[:o, :i] = w.float()
    blocks = wp.view(ob, block, ib, block)
    amax = blocks.abs().amax((1, 3)).clamp_min(1e-12)
    sb = e8m0_encode_ceil(amax / E4M3_MAX)
    scale = e8m0_decode(sb)
    q = e4m3_encode(blocks / scale[:, None, :, None]).view(ob * block, ib * block)[:o, :i].contiguous()
    return q, sb


def weight_dequant_fp8_block(q: torch.Tensor, sb: torch.Tensor, block: int = 128) -> torch.Tensor:
    o, i = q.shape
    scale = e8m0_decode(sb).repeat_interleave(block, 0)[:o].repeat_interleave(block, 1)[:, :i]
    return e4m3_decode(q) * scale


def weight_quant_mxfp4(w: torch.Tensor, group: int = 32) -> Tuple[torch.Tensor, torch.Tensor]:
    """[out, in] -> (packed bytes [out, in/2], e8m0 scales [out, in/group])."""
    o, i = w.shape
    assert i % group == 0
    g = w.float().view(o, i // group, group)
    amax = g.abs().amax(-1).clamp_min(1e-12)
    sb = e8m0_encode_ceil(amax / FP4_MAX)
    packed = fp4_pack((g / e8m0_decode(sb).unsqueeze(-1)).view(o, i))
    return packed, sb


def weight_dequant_mxfp4(packed: torch.Tensor, sb: torch.Tensor, group: int = 32) -> torch.Tensor:
    o = packed.shape[0]
    v = fp4_unpack(packed)
    i = v.shape[1]
    return (v.view(o, i // group, group) * e8m0_decode(sb).unsqueeze(-1)).view(o, i)


# ---------------------------------------------------------------------------------------- QAT + Hadamard
def bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).float()


def fp8_qat(x: torch.Tensor, block: int = 128) -> torch.Tensor:
    """Quantise to FP8 per 1 x block and come back, with the bf16 write-back the device path has."""
    q, sb = act_quant_fp8(x, block)
    return bf16_round(act_dequant_fp8(q, sb, block))


def fp4_qat(x: torch.Tensor, group: int = 32) -> torch.Tensor:
    *lead, n = x.shape
    p, sb = weight_quant_mxfp4(x.reshape(-1, n), group)
    return bf16_round(weight_dequant_mxfp4(p, sb, group)).reshape(*lead, n)


def hadamard(x: torch.Tensor) -> torch.Tensor:
    """Orthonormal fast Walsh-Hadamard transform over the last dim (power of two), scale n^-1/2."""
    n = x.shape[-1]
    assert n & (n - 1) == 0, "Hadamard length must be a power of two"
    y = x.float().clone()
    h = 1
    while h < n:
        y = y.view(*x.shape[:-1], n // (2 * h), 2, h)
        a, b = y[..., 0, :], y[..., 1, :]
        y = torch.stack((a + b, a - b), dim=-2).reshape(*x.shape[:-1], n)
        h *= 2
    return y * (n ** -0.5)
