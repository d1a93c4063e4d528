"""Weight quantisation helpers (torch): group-wise asymmetric int4 / int8 in the IR layout.

IR layout of a compressed FullyConnected weight (the pattern the reference recognises in
src/common/transformations/src/transformations/pattern_blocks/compressed_weights_block.cpp):
``Constant(u4) [N, G, gs] -> Convert(f16) -> Subtract(Convert(Constant(u4) [N, G, 1])) ->
Multiply(Constant(f16) [N, G, 1]) -> Reshape [N, K]``; sub-byte elements are packed LSB first
(element 2i in bits 0..3 of byte i, element 2i+1 in bits 4..7;
src/core/dev_api/openvino/core/type/element_iterator.hpp).
"""
from __future__ import annotations

import torch


def pack_u4(vals: torch.Tensor) -> torch.Tensor:
    """uint8 values in [0, 15], any shape with an even number of elements -> packed bytes (flat)."""
    v = vals.reshape(-1).to(torch.uint8)
    assert v.numel() % 2 == 0
    return (v[0::2] | (v[1::2] << 4)).contiguous()


def unpack_u4(packed: torch.Tensor, numel: int) -> torch.Tensor:
    p = packed.reshape(-1)
    out = torch.empty(p.numel() * 2, dtype=torch.uint8, device=p.device)
    out[0::2] = p & 0xF
    out[1::2] = p >> 4
    return out[:numel]


def quantize_u4_asym(w: torch.Tensor, group_size: int = 128):
    """w [N, K] float -> (q uint8 [N, K] in 0..15, scale fp16 [N, G], zp uint8 [N, G])."""
    N, K = w.shape
    assert K % group_size == 0
    G = K // group_size
    wg = w.float().reshape(N, G, group_size)
    mn = wg.amin(dim=2, keepdim=True)
    mx = wg.amax(dim=2, keepdim=True)
    scale = ((mx - mn) / 15.0).clamp_min(1e-8)
    scale = scale.to(torch.float16).float().clamp_min(6e-8)
    zp = torch.round(-mn / scale).clamp(0, 15)
    q = torch.round(wg / scale + zp).clamp(0, 15)
    return (q.reshape(N, K).to(torch.uint8), scale.reshape(N, G).to(torch.float16), zp.reshape(N, G).to(torch.uint8))


def dequantize_u4(q: torch.Tensor, scale: torch.Tensor, zp: torch.Tensor, group_size: int) -> torch.Tensor:
    N, K = q.shape
    G = K // group_size
    return ((q.float().reshape(N, G, group_size) - zp.float().reshape(N, G, 1)) * scale.float().reshape(N, G, 1)).reshape(N, K)


def quantize_u8_asym(w: torch.Tensor, group_size: int):
    N, K = w.shape
    G = K // group_size
    wg = w.float().reshape(N, G, group_size)
    mn = wg.amin(dim=2, keepdim=True)
    mx = wg.amax(dim=2, keepdim=True)
    scale = ((mx - mn) / 255.0).to(torch.float16).float().clamp_min(6e-8)
    zp = torch.round(-mn / scale).clamp(0, 255)
    q = torch.round(wg / scale + zp).clamp(0, 255)
    return (q.reshape(N, K).to(torch.uint8), scale.reshape(N, G).to(torch.float16), zp.reshape(N, G).to(torch.uint8))


def random_u4_weight(N: int, K: int, group_size: int, device, seed: int = 0, std: float = 0.02):
    """Random compressed weight without materialising the float matrix: uniform nibbles, zero point 8
    +-1, scale chosen so that the dequantised weights have roughly the requested std."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    G = K // group_size
    packed = torch.randint(0, 256, (N * K // 2,), dtype=torch.uint8, device=device, generator=g)
    zp = torch.randint(7, 10, (N, G), dtype=torch.uint8, device=device, generator=g)
    # uniform 0..15 has std ~4.6
    scale = (torch.rand((N, G), device=device, generator=g) * 0.5 + 0.75) * (std / 4.6)
    return packed, scale.to(torch.float16), zp


def quantize_f8_block(w: torch.Tensor, block: int = 128):
    """Float [N, K] -> (fp8 e4m3 values [N, K] as uint8, fp32 scales [ceil(N/block), K/block]); every block x block tile
    is scaled so that its largest magnitude maps to 448 (the e4m3 maximum). Scales are rounded to bf16 precision so that
    kernels which apply them in bf16 reproduce them exactly."""
    N, K = w.shape
    assert K % block == 0
    nb = (N + block - 1) // block
    pad = nb * block - N
    wf = torch.nn.functional.pad(w.float(), (0, 0, 0, pad)) if pad else w.float()
    tiles = wf.reshape(nb, block, K // block, block)
    amax = tiles.abs().amax(dim=(1, 3)).clamp_min(1e-12)                 # [nb, K/block]
    scale = (amax / 448.0).to(torch.bfloat16).float()
    q = (tiles / scale[:, None, :, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    q = q.reshape(nb * block, K)[:N].contiguous()
    return q.view(torch.uint8), scale


def dequantize_f8_block(q: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    N, K = q.shape
    w = q.view(torch.float8_e4m3fn).float()
    s = scale.repeat_interleave(block, dim=0)[:N].repeat_interleave(block, dim=1)
    return w * s
