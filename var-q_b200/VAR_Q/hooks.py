"""The cache section of the VAR and Infinity ``SelfAttention.forward`` hooks, on the fused route.

The reference builds two ``VAR_Q`` objects per attention layer in ``kv_caching(True)`` and, at
every scale step, runs ``k = k_quant.use_var_q(k); v = v_quant.use_var_q(v)`` followed by a cast
and flash-attn / SDPA (VAR/models/basic_var.py:104-117,143-162;
Infinity/infinity/models/basic.py:254-271,327-351).  ``LayerKV`` owns the same pair of quantizers
and replaces those lines by ``append`` + one attention call over the packed cache:

    # kv_caching(True)
    self.kv = LayerKV.from_module(self)          # reads q_bits, quant_method, qkv_format, block_idx
    # forward, where the reference has "Implement VAR-Q here"
    oup = self.kv.step(q, k, v, softmax_scale=self.scale, out_dtype=main_type).view(B, L, C)
    # kv_caching(False)
    self.kv = None

``step`` takes q, k, v in the layer's own layout ('BLHc' on the flash/xformers path, 'BHLc'
otherwise; k and v may be strided views of the fused QKV activation) and returns ``[B, L, H, c]``.
"""
from typing import Any, Dict, Optional

import torch

from .attention import attend
from .quant import VAR_Q


class LayerKV:
    """Packed K and V caches of one attention layer."""

    def __init__(self, q_bits: int = 8, quant_method: str = 'G_SCALE_HEAD_DIM', qkv_format: str = 'BLHc',
                 blk_idx: int = 0, k_kwargs: Optional[Dict[str, Any]] = None,
                 v_kwargs: Optional[Dict[str, Any]] = None, max_tokens: Optional[int] = None):
        base = dict(quant_bits=q_bits, qkv_format=qkv_format, quant_method=quant_method)
        kk, vk = dict(base), dict(base)
        kk.update(k_kwargs or {})
        vk.update(v_kwargs or {})
        self.k_quant = VAR_Q(blk_idx=blk_idx, max_tokens=max_tokens, **kk)
        self.v_quant = VAR_Q(blk_idx=blk_idx, max_tokens=max_tokens, **vk)

    @classmethod
    def from_module(cls, module, **overrides) -> Optional["LayerKV"]:
        """Build from the attributes both reference ``SelfAttention`` classes carry
        (VAR/models/basic_var.py:79-83; Infinity/infinity/models/basic.py:245-249);
        returns None when ``enable_quantization`` is off, like the reference's ``k_quant = None``."""
        if not getattr(module, 'enable_quantization', False):
            return None
        return cls(q_bits=module.q_bits, quant_method=module.quant_method, qkv_format=module.qkv_format,
                   blk_idx=getattr(module, 'block_idx', 0), **overrides)

    @classmethod
    def from_config(cls, config, qkv_format: Optional[str] = None, blk_idx: int = 0, max_tokens=None):
        """Build from a ``VARQConfig`` (per-K / per-V settings and method aliases resolved)."""
        k, v = config.get_quantizer_kwargs('k'), config.get_quantizer_kwargs('v')
        if k is None:
            return None
        fmt = qkv_format or k.get('qkv_format', 'BLHc')
        strip = lambda d: {n: x for n, x in d.items() if n not in ('quant_bits', 'quant_method', 'qkv_format')}
        self = cls.__new__(cls)
        self.k_quant = VAR_Q(quant_bits=k['quant_bits'], qkv_format=fmt, quant_method=k['quant_method'],
                             blk_idx=blk_idx, max_tokens=max_tokens, **strip(k))
        self.v_quant = VAR_Q(quant_bits=v['quant_bits'], qkv_format=fmt, quant_method=v['quant_method'],
                             blk_idx=blk_idx, max_tokens=max_tokens, **strip(v))
        return self

    def set_format(self, qkv_format: str):
        """Infinity assigns the layout at every forward (Infinity/infinity/models/basic.py:309,314)."""
        self.k_quant.qkv_format = self.v_quant.qkv_format = qkv_format

    @property
    def n_tokens(self) -> int:
        return self.k_quant.n_tokens

    def step(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float,
             out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """Quantize+append this scale's K and V, attend q over everything cached: ``[B, L, H, c]``."""
        return attend(q, k, v, self.k_quant, self.v_quant, softmax_scale, out_dtype)

    def step_reference_route(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float,
                             main_type: torch.dtype) -> torch.Tensor:
        """The reference's sequence on the same kernels: fp32 ``use_var_q`` outputs, cast, SDPA.
        Kept for A/B checks of the fused route; returns ``[B, L, H, c]``."""
        kd = self.k_quant.use_var_q(k).to(main_type)
        vd = self.v_quant.use_var_q(v).to(main_type)
        q = q.to(main_type)
        if self.k_quant.qkv_format == 'BLHc':
            q, kd, vd = (t.transpose(1, 2) for t in (q, kd, vd))
        o = torch.nn.functional.scaled_dot_product_attention(q, kd, vd, scale=softmax_scale)
        return o.transpose(1, 2).contiguous()
