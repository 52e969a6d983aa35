"""NVFP4 weight preparation and routing index with the reference's surface
(python/nvfp4_gemm/layout.py there): same names, shapes, dtypes and errors.

``quantize_weight_nvfp4`` runs the native CUDA quantiser for CUDA tensors (the
product path; it raises if the compiled library is missing).  Like the reference,
which computes on whatever device the tensor lives on, a CPU tensor is quantised on
the CPU with torch ops; that branch is the host-tensor behaviour of the API, never a
substitute for the CUDA path.
"""
from __future__ import annotations

import torch

BLOCK_SIZE = 16
K_PER_SF_ATOM = 64
E2M1_MAX = 6.0
E4M3_MAX = 448.0
E4M3_MIN_SUBNORMAL = 2.0 ** -9

_LEVELS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def quantize_e2m1_codes(x: torch.Tensor) -> torch.Tensor:
    """RNE onto the E2M1 grid; 4-bit codes as uint8, sign bit from signbit(x).

    The grid {0, .5, 1, 1.5, 2, 3, 4, 6} has one mantissa bit, so for magnitudes
    below 1 the step is 0.5, then 0.5, 1, 2 per binade: rounding the magnitude
    divided by its step to the nearest even integer is RNE on the grid.
    """
    x = x.to(torch.float32)
    mag = x.abs()
    step = torch.where(mag < 2.0, torch.full_like(mag, 0.5),
                       torch.where(mag < 4.0, torch.full_like(mag, 1.0), torch.full_like(mag, 2.0)))
    q = torch.clamp(torch.round(mag / step) * step, max=E2M1_MAX)        # torch.round is half-to-even
    q = torch.where(torch.isfinite(mag), q, torch.full_like(q, E2M1_MAX))
    code = torch.bucketize(q, torch.tensor(_LEVELS, device=x.device)).to(torch.uint8)
    return code | (torch.signbit(x).to(torch.uint8) << 3)


def pack_e2m1_pairs(codes: torch.Tensor) -> torch.Tensor:
    """Two 4-bit codes per byte along the last axis, element 2i in the low nibble."""
    if codes.shape[-1] % 2 != 0:
        raise ValueError("last dim must be even to pack FP4 pairs")
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).to(torch.int8)


def pack_sf_atoms(s_codes: torch.Tensor) -> torch.Tensor:
    """(E, N, K/16) E4M3 bytes -> (E*K/64, N) int32, byte j of a word = 16-block j of the atom."""
    e, n, nb = s_codes.shape
    if nb % 4 != 0:
        raise ValueError("K // 16 must be a multiple of 4 (one atom = 4 sub-blocks)")
    w = s_codes.reshape(e, n, nb // 4, 4).to(torch.int32)
    packed = w[..., 0] | (w[..., 1] << 8) | (w[..., 2] << 16) | (w[..., 3] << 24)
    return packed.permute(0, 2, 1).reshape(e * (nb // 4), n).contiguous()


def _quantize_weight_host(w: torch.Tensor):
    e, n, k = w.shape
    w32 = w.to(torch.float32)
    tiny = torch.finfo(torch.float32).tiny
    gw = torch.clamp(w32.reshape(e, -1).abs().amax(dim=-1) / (E4M3_MAX * E2M1_MAX), min=tiny)
    blocks = w32.reshape(e, n, k // BLOCK_SIZE, BLOCK_SIZE)
    s_pre = (blocks.abs().amax(dim=-1) / E2M1_MAX) / gw.reshape(-1, 1, 1)
    s8 = torch.clamp(s_pre, min=E4M3_MIN_SUBNORMAL).to(torch.float8_e4m3fn)
    denom = torch.clamp(s8.to(torch.float32).unsqueeze(-1) * gw.reshape(-1, 1, 1, 1), min=tiny)
    codes = quantize_e2m1_codes(blocks / denom).reshape(e, n, k)
    return pack_e2m1_pairs(codes).reshape(e * n, k // 2).contiguous(), pack_sf_atoms(s8.view(torch.uint8)), gw.contiguous()


def quantize_weight_nvfp4(w: torch.Tensor):
    """(E, N, K) BF16/FP32 -> b int8 (E*N, K/2), sfb int32 (E*K/64, N), gw fp32 (E,)."""
    if w.dim() != 3:
        raise ValueError("expected weights shaped (E, N, K)")
    k = w.shape[2]
    if k % K_PER_SF_ATOM != 0:
        raise ValueError(f"K={k} must be a multiple of {K_PER_SF_ATOM}")
    if w.is_cuda:
        from . import _C
        return _C.quantize_weight(w)
    return _quantize_weight_host(w)


def load_checkpoint_weights_nvfp4(parts, global_scale_is_divisor: bool = True):
    """NVFP4 checkpoint tensors -> (b, sfb, gw) for the grouped GEMM, on the GPU.

    ``parts``: the projections to fuse along N, in order, each a triple (weight_packed uint8 (E, rows, K/2),
    weight_scale float8_e4m3fn / uint8 (E, rows, K/16), weight_global_scale float32 (E,)) stacked over the experts:
    [gate, up] for a fused gate+up projection, [down] for a down projection.  Projections with different global
    scales get one shared gw per expert and re-folded block scales, the integration step the reference describes
    and leaves to the weight loader (docs/bf16-dual-nvfp4-algorithm.html:235-244 there).  CUDA tensors only.
    """
    for part in parts:
        if not all(t.is_cuda for t in part):
            raise RuntimeError("load_checkpoint_weights_nvfp4 runs on the GPU: move the checkpoint tensors to a CUDA device")
    from . import _C
    return _C.load_checkpoint_weights(parts, global_scale_is_divisor)


def unpack_sf_atoms(sfb: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Inverse of pack_sf_atoms: (E*K/64, N) int32 -> (E, N, K/16) E4M3 bytes (the checkpoint's weight_scale layout)."""
    atoms = sfb.shape[0] // num_experts
    n = sfb.shape[1]
    words = sfb.reshape(num_experts, atoms, n).permute(0, 2, 1).contiguous()
    return words.view(torch.uint8).reshape(num_experts, n, atoms * 4)


def dequantize_weight_nvfp4(b, sfb, gw, num_experts: int, n: int, k: int) -> torch.Tensor:
    """Inverse of quantize_weight_nvfp4: FP32 (E, N, K) = dec(q) * dec(S) * G."""
    u = b.reshape(num_experts, n, k // 2).view(torch.uint8)
    codes = torch.stack([u & 0xF, u >> 4], dim=-1).reshape(num_experts, n, k).long()
    mag = torch.tensor(_LEVELS, device=b.device)[codes & 7]
    vals = torch.where((codes & 8) != 0, -mag, mag)
    atoms = k // K_PER_SF_ATOM
    words = sfb.reshape(num_experts, atoms, n).permute(0, 2, 1).contiguous()
    s = words.view(torch.uint8).reshape(num_experts, n, atoms * 4).view(torch.float8_e4m3fn).to(torch.float32)
    return vals * s.repeat_interleave(BLOCK_SIZE, dim=-1) * gw.reshape(-1, 1, 1).to(torch.float32)


def make_m_indices(group_sizes, device=None, alignment: int = 128) -> torch.Tensor:
    """Expert id per row; every group size must be a multiple of ``alignment``."""
    sizes = torch.as_tensor(group_sizes, dtype=torch.int64)
    bad = torch.nonzero(sizes % alignment != 0).flatten()
    if bad.numel():
        i = int(bad[0])
        raise ValueError(f"group {i} has {int(sizes[i])} rows; each must be a multiple of {alignment}")
    out = torch.repeat_interleave(torch.arange(sizes.numel(), dtype=torch.int32), sizes)
    return out.to(device) if device is not None else out
