"""Quantizers that write ggml block bytes (torch, CPU or CUDA tensors), used to make synthetic GGUF models.

q4_0 / q5_0 / q8_0 follow ggml's reference quantizers (the ones `llama-quantize --pure` and the reference's tools/convert/quantize_q4_0.py:42-52 apply through
gguf-py): the element of largest magnitude in a block of 32 fixes the scale. q4_K and q6_K are this project's own simple quantizers: they emit valid blocks
(any valid block bytes are a legitimate model; parity is defined on the decoder given the bytes), not ggml's error-minimizing search.
Every function takes a float32 tensor [rows, cols] and returns a uint8 tensor [rows, cols / block * block_bytes].
"""
from __future__ import annotations

import torch

from . import _lib as L


def _f16_bytes(x: torch.Tensor) -> torch.Tensor:
    """[..., n] float -> [..., n, 2] uint8 (little-endian f16)."""
    return x.to(torch.float16).contiguous().view(torch.uint8).reshape(*x.shape, 2)


def quantize_q4_0(x: torch.Tensor) -> torch.Tensor:
    rows, cols = x.shape
    b = x.reshape(rows, cols // 32, 32).float()
    idx = b.abs().argmax(dim=-1, keepdim=True)            # first element of largest magnitude
    mx = b.gather(-1, idx)
    d = mx / -8.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = (b * inv + 8.5).to(torch.int32).clamp_(max=15).to(torch.uint8)       # truncation of a non-negative number
    qs = q[..., :16] | (q[..., 16:] << 4)
    return torch.cat([_f16_bytes(d.squeeze(-1)), qs], dim=-1).reshape(rows, -1)


def quantize_q5_0(x: torch.Tensor) -> torch.Tensor:
    rows, cols = x.shape
    b = x.reshape(rows, cols // 32, 32).float()
    idx = b.abs().argmax(dim=-1, keepdim=True)
    mx = b.gather(-1, idx)
    d = mx / -16.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = (b * inv + 16.5).to(torch.int32).clamp_(max=31)
    lo, hi = q[..., :16], q[..., 16:]
    qs = ((lo & 15) | ((hi & 15) << 4)).to(torch.uint8)
    shifts = torch.arange(16, device=x.device, dtype=torch.int64)
    qh = (((lo >> 4) & 1).to(torch.int64) << shifts).sum(-1) | (((hi >> 4) & 1).to(torch.int64) << (shifts + 16)).sum(-1)
    qh_bytes = torch.stack([(qh >> (8 * i)) & 0xFF for i in range(4)], dim=-1).to(torch.uint8)
    return torch.cat([_f16_bytes(d.squeeze(-1)), qh_bytes, qs], dim=-1).reshape(rows, -1)


def quantize_q8_0(x: torch.Tensor) -> torch.Tensor:
    rows, cols = x.shape
    b = x.reshape(rows, cols // 32, 32).float()
    d = b.abs().amax(dim=-1, keepdim=True) / 127.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    v = b * inv
    q = torch.where(v >= 0, torch.floor(v + 0.5), torch.ceil(v - 0.5)).to(torch.int8)      # roundf: halves away from zero
    return torch.cat([_f16_bytes(d.squeeze(-1)), q.view(torch.uint8)], dim=-1).reshape(rows, -1)


def quantize_q4_k(x: torch.Tensor) -> torch.Tensor:
    rows, cols = x.shape
    b = x.reshape(rows, cols // 256, 8, 32).float()
    mn = (-b.amin(dim=-1)).clamp_(min=0)                  # offset of each sub-block, >= 0
    sc = (b.amax(dim=-1) + mn) / 15.0                     # step of each sub-block
    d = _to_half(sc.amax(dim=-1, keepdim=True) / 63.0)
    dmin = _to_half(mn.amax(dim=-1, keepdim=True) / 63.0)
    isc = torch.where(d > 0, torch.round(sc / d), torch.zeros_like(sc)).clamp_(0, 63).to(torch.int32)
    imn = torch.where(dmin > 0, torch.round(mn / dmin), torch.zeros_like(mn)).clamp_(0, 63).to(torch.int32)
    step = (d * isc).unsqueeze(-1)
    off = (dmin * imn).unsqueeze(-1)
    q = torch.where(step > 0, torch.round((b + off) / step), torch.zeros_like(b)).clamp_(0, 15).to(torch.uint8)
    scales = torch.empty(rows, cols // 256, 12, dtype=torch.uint8, device=x.device)       # ggml's 6-bit packing, the inverse of get_scale_min_k4
    for j in range(4):
        scales[..., j] = (isc[..., j] | ((isc[..., j + 4] >> 4) << 6)).to(torch.uint8)
        scales[..., j + 4] = (imn[..., j] | ((imn[..., j + 4] >> 4) << 6)).to(torch.uint8)
        scales[..., j + 8] = ((isc[..., j + 4] & 15) | ((imn[..., j + 4] & 15) << 4)).to(torch.uint8)
    qs = (q[..., 0::2, :] | (q[..., 1::2, :] << 4)).reshape(rows, cols // 256, 128)      # byte 32p + l: low nibble sub-block 2p, high 2p + 1
    return torch.cat([_f16_bytes(d.squeeze(-1)), _f16_bytes(dmin.squeeze(-1)), scales, qs], dim=-1).reshape(rows, -1)


def quantize_q6_k(x: torch.Tensor) -> torch.Tensor:
    rows, cols = x.shape
    b = x.reshape(rows, cols // 256, 16, 16).float()
    sub = b.abs().amax(dim=-1) / 31.0                     # step of each 16-element sub-block
    d = _to_half(sub.amax(dim=-1, keepdim=True) / 127.0)
    isc = torch.where(d > 0, torch.round(sub / d), torch.zeros_like(sub)).clamp_(0, 127).to(torch.int32)
    step = (d * isc).unsqueeze(-1)
    q = (torch.where(step > 0, torch.round(b / step), torch.zeros_like(b)).clamp_(-32, 31) + 32).to(torch.uint8).reshape(rows, cols // 256, 2, 4, 32)
    # element 128h + 32k + l: low nibble in ql[64h + 32(k & 1) + l] (low half for k < 2, high half otherwise), bits 4..5 in qh[32h + l] at bit 2k
    lo = q & 15
    ql = torch.cat([lo[..., 0, :] | (lo[..., 2, :] << 4), lo[..., 1, :] | (lo[..., 3, :] << 4)], dim=-1).reshape(rows, cols // 256, 128)
    hi = q >> 4
    qh = (hi[..., 0, :] | (hi[..., 1, :] << 2) | (hi[..., 2, :] << 4) | (hi[..., 3, :] << 6)).reshape(rows, cols // 256, 64)
    # the scale of element 128h + 32k + l is scales[8h + 2k + l / 16]; sub-block s = 8h + 2k + l / 16 holds elements 16 s .. 16 s + 15, the natural order
    return torch.cat([ql, qh, isc.to(torch.int8).view(torch.uint8), _f16_bytes(d.squeeze(-1))], dim=-1).reshape(rows, -1)


def _to_half(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16).float()


def to_f16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16).contiguous().view(torch.uint8).reshape(x.shape[0], -1)


QUANTIZERS = {L.F16: to_f16, L.Q4_0: quantize_q4_0, L.Q5_0: quantize_q5_0, L.Q8_0: quantize_q8_0, L.Q4_K: quantize_q4_k, L.Q6_K: quantize_q6_k}


def quantize(dtype: int, x: torch.Tensor) -> torch.Tensor:
    if x.shape[1] % L.BLOCK_ELEMS[dtype] != 0:
        raise ValueError(f"rows of {x.shape[1]} elements are not whole {L.DTYPE_NAMES[dtype]} blocks")
    return QUANTIZERS[dtype](x)
