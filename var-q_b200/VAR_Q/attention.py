"""Attention straight from the packed KV cache.

Replaces the reference's ``use_var_q`` -> fp32 ``dequant_all`` -> cast -> attention-library
sequence (VAR/models/basic_var.py:143-162; Infinity/infinity/models/basic.py:327-351) by
``append`` (one fused quantize+pack launch per tensor) and one ``varq_attn_fwd`` call that
dequantises K/V tiles on chip.
"""
from typing import Optional

import torch

from . import _cabi
from .quant import VAR_Q


def attend_cached(q: torch.Tensor, k_quant: VAR_Q, v_quant: VAR_Q, softmax_scale: float,
                  out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """softmax(q K^T * scale) V over the committed caches; no mask.

    ``q`` is in the quantizers' ``qkv_format``.  Returns ``[B, Lq, H, c]`` (contiguous), which
    both hook sites immediately view as ``[B, Lq, H*c]``.
    """
    _cabi.require_cuda(q, "q")
    if k_quant.n_tokens == 0 or k_quant.n_tokens != v_quant.n_tokens:
        raise ValueError("[VAR-Q]: K and V caches must hold the same, non-zero number of tokens")
    if q.dtype not in _cabi.DTYPES:
        q = q.to(torch.float32)
    if q.stride(-1) != 1:
        q = q.contiguous()
    fmt = k_quant.qkv_format
    B, D = q.size(0), q.size(3)
    Lq, H = (q.size(1), q.size(2)) if fmt == 'BLHc' else (q.size(2), q.size(1))
    if (B, H, D) != k_quant._shape or (B, H, D) != v_quant._shape:
        raise ValueError(f"[VAR-Q]: q (B,H,c)={(B, H, D)} does not match the cache {k_quant._shape}")
    out_dtype = out_dtype or (q.dtype if q.dtype != torch.float32 else torch.float32)
    out = torch.empty((B, Lq, H, D), dtype=out_dtype, device=q.device)
    kc, kp = k_quant.cache_descriptors()
    vc, vp = v_quant.cache_descriptors()
    lib = _cabi.lib()
    Lk = k_quant.n_tokens
    ws_bytes = lib.varq_attn_workspace_bytes(B, H, Lq, Lk, D, k_quant.store_bits, v_quant.store_bits)
    ws = _cabi.workspace(q.device, ws_bytes) if ws_bytes else None
    qd = k_quant._item_desc(q)
    od = _cabi.tensor_desc(out.data_ptr(), _cabi.DTYPES[out_dtype], Lq * H * D, H * D, D)
    with torch.cuda.device(q.device):
        rc = lib.varq_attn_fwd(qd, kc, vc, kp, vp, B, H, Lq, Lk, D, k_quant.store_bits, v_quant.store_bits,
                               float(softmax_scale), od, ws.data_ptr() if ws is not None else None, ws_bytes,
                               _cabi.stream_ptr(q.device))
    _cabi.check(rc)
    return out


def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_quant: VAR_Q, v_quant: VAR_Q,
           softmax_scale: float, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Quantize and append this step's K and V, then attend over everything cached."""
    k_quant.append(k)
    v_quant.append(v)
    return attend_cached(q, k_quant, v_quant, softmax_scale, out_dtype)
