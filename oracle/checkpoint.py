"""TEST INFRASTRUCTURE -- CPU restatement of the checkpoint weight loader (not product code).

The reference describes the step and leaves it to "the real weight loader"
(docs/bf16-dual-nvfp4-algorithm.html:235-244 there): projections stored separately, each with its own
``weight_global_scale``, are fused along N under one shared per-expert scale gw' and every E4M3 block scale is
re-quantised to S' = Q_e4m3(S * (G_p / gw')).  There is no reference code for it, so parity for this function is
pinned only through what it shares with the pinned functions (the E4M3 rounding of ``oracle.e4m3_encode``, the
physical layouts of python/nvfp4_gemm/layout.py:108-127) and through the round trip of a single part, which must
return the checkpoint's own bytes.  The rule stated here is the one the CUDA loader implements:

    G_p[e]  = 1 / global_p[e]  (divisor convention)  or  global_p[e]      (one FP32 division)
    gw'[e]  = max_p G_p[e]
    ratio   = G_p[e] / gw'[e]                                             (one FP32 division, <= 1)
    S'      = RNE_e4m3(dec(S) * ratio); a non-zero S whose product rounds to zero becomes the smallest subnormal
"""
from __future__ import annotations

import numpy as np
import torch

from . import e4m3_decode, e4m3_encode


def load_checkpoint_weights(parts, global_scale_is_divisor: bool = True):
    """parts: list of (weight_packed uint8 (E, rows, K/2), weight_scale uint8 (E, rows, K/16), global f32 (E,)).
    Returns b int8 (E*N, K/2), sfb int32 (E*K/64, N), gw float32 (E,) as CPU tensors."""
    mult = []
    for _, _, g in parts:
        g = g.detach().cpu().reshape(-1).to(torch.float32).numpy()
        mult.append((np.float32(1.0) / g).astype(np.float32) if global_scale_is_divisor else g.astype(np.float32))
    gw = np.maximum.reduce(mult).astype(np.float32)
    codes, scales = [], []
    for (wp, ws, _), g in zip(parts, mult):
        wp = wp.detach().cpu().contiguous().view(torch.uint8)
        ws = ws.detach().cpu().contiguous().view(torch.uint8)
        ratio = (g / gw).astype(np.float32)                                   # (E,)
        mag = ws & 0x7F
        dec = e4m3_decode(mag).numpy().astype(np.float32)
        folded = e4m3_encode(torch.from_numpy((dec * ratio[:, None, None]).astype(np.float32)))
        folded = torch.where((folded == 0) & (mag != 0), torch.ones_like(folded), folded)
        codes.append(wp)
        scales.append(folded)
    packed = torch.cat(codes, dim=1)                                          # (E, N, K/2)
    sc = torch.cat(scales, dim=1)                                             # (E, N, K/16)
    e, n, nb = sc.shape
    w = sc.reshape(e, n, nb // 4, 4).to(torch.int32)
    words = w[..., 0] | (w[..., 1] << 8) | (w[..., 2] << 16) | (w[..., 3] << 24)
    sfb = words.permute(0, 2, 1).reshape(e * (nb // 4), n).contiguous()
    return packed.reshape(e * n, -1).view(torch.int8).contiguous(), sfb, torch.from_numpy(gw.copy())
