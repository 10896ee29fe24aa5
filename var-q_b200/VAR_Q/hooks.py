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

from . import _cabi
from .attention import attend, attend_cached
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


# ---------------------------------------------------------------------- fused producer + install helper
def _strided_desc(t: torch.Tensor, fmt: str) -> _cabi.Tensor:
    sb, s1, s2, sd = t.stride()
    if sd != 1:
        raise ValueError("[VAR-Q]: the last dim of q / k / v must be contiguous")
    sl, sh = (s1, s2) if fmt == 'BLHc' else (s2, s1)
    return _cabi.tensor_desc(t.data_ptr(), _cabi.DTYPES[t.dtype], sb, sl, sh)


def normalise_qk(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_quant: VAR_Q, v_quant: VAR_Q,
                 scale_mul: Optional[torch.Tensor] = None, eps: float = 1e-12):
    """One kernel for the producer side of the hook: ``q = normalize(q) * scale_mul``, ``k = normalize(k)`` in fp32
    (VAR/models/basic_var.py:137-141; Infinity/infinity/models/basic.py:316-320) and, for quantizers whose statistics
    are shared over batch and tokens (per-dim, per-step), the min / max tables of the normalised k and of v, so that
    their quantize call reads K / V only once more.  q, k, v are views in the quantizers' layout (strided views of the
    fused QKV activation are fine); ``scale_mul`` holds one factor per head.  Returns ``(q, k, k_stats, v_stats)``;
    a statistics entry is None when that quantizer has no use for it."""
    fmt = k_quant.qkv_format
    _cabi.require_cuda(q, "q")
    B, D = q.size(0), q.size(3)
    L, H = (q.size(1), q.size(2)) if fmt == 'BLHc' else (q.size(2), q.size(1))
    q_out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    k_out = torch.empty(k.shape, dtype=torch.float32, device=q.device)
    lib = _cabi.lib()
    kg, vg = k_quant.column_grouping(D), v_quant.column_grouping(D)

    def table(g):
        if g is None:
            return None
        nbytes = lib.varq_quant_workspace_bytes(B, L, H, D, _cabi.F32, 8, g)
        return torch.empty(max(nbytes, 8), dtype=torch.uint8, device=q.device)
    k_stats, v_stats = table(kg), table(vg)
    sm = None
    if scale_mul is not None:
        sm = scale_mul.detach().to(device=q.device, dtype=torch.float32).reshape(-1).contiguous()
        if sm.numel() != H:
            raise ValueError(f"[VAR-Q]: scale_mul must hold one factor per head ({H}), got {sm.numel()}")
    with torch.cuda.device(q.device):
        rc = lib.varq_qk_norm_stats(
            _strided_desc(q, fmt), _strided_desc(k, fmt), _strided_desc(v, fmt) if vg is not None else None,
            B, L, H, D, sm.data_ptr() if sm is not None else None, float(eps),
            _strided_desc(q_out, fmt), _strided_desc(k_out, fmt),
            kg, k_stats.data_ptr() if k_stats is not None else None,
            vg, v_stats.data_ptr() if v_stats is not None else None, _cabi.stream_ptr(q.device))
    _cabi.check(rc)
    return q_out, k_out, k_stats, v_stats


def _step_normalised(self, q, k, v, scale_mul, softmax_scale, out_dtype=None):
    """``LayerKV.step`` with the L2-normalisation of q and k (and the statistics pass of column groupings) fused in front."""
    qn, kn, ks, vs = normalise_qk(q, k, v, self.k_quant, self.v_quant, scale_mul)
    self.k_quant.append(kn, ks)
    self.v_quant.append(v, vs)
    return attend_cached(qn, self.k_quant, self.v_quant, softmax_scale, out_dtype)


LayerKV.step_normalised = _step_normalised


def install(attn: torch.nn.Module, max_tokens: Optional[int] = None, k_kwargs=None, v_kwargs=None) -> torch.nn.Module:
    """Put the fused route into a VAR-style ``SelfAttention`` module without editing its source file.

    The module must carry what the reference class does (VAR/models/basic_var.py:73-117): ``mat_qkv``, ``q_bias``,
    ``zero_k_bias``, ``v_bias``, ``proj``, ``proj_drop``, ``num_heads``, ``head_dim``, ``scale``, ``attn_l2_norm``
    (with ``scale_mul_1H11`` / ``max_scale_mul``), ``caching``, ``enable_quantization``, ``q_bits``, ``quant_method``,
    ``block_idx``.  ``kv_caching(True)`` then builds a ``LayerKV`` instead of two ``VAR_Q`` objects, and ``forward``
    takes the packed-cache route while caching with quantization is on (any other call goes to the original
    ``forward``).  The layout is BLHc whatever the module would pick: the kernels read q, k, v as strided views of the
    fused QKV activation, so no permute or copy is needed.  Returns the module.
    """
    import types
    cls_forward, cls_caching = type(attn).forward, type(attn).kv_caching

    def kv_caching(self, enable: bool):
        cls_caching(self, enable)
        self._varq_kv = None
        if enable and getattr(self, 'enable_quantization', False):
            self.k_quant = self.v_quant = None          # the reference's pair is not used on this route
            self._varq_kv = LayerKV(q_bits=self.q_bits, quant_method=self.quant_method, qkv_format='BLHc',
                                    blk_idx=getattr(self, 'block_idx', 0), k_kwargs=k_kwargs, v_kwargs=v_kwargs,
                                    max_tokens=max_tokens)

    def forward(self, x, attn_bias=None):
        kv = getattr(self, '_varq_kv', None)
        if kv is None or not self.caching:
            return cls_forward(self, x, attn_bias)
        B, L, C = x.shape
        bias = torch.cat((self.q_bias, self.zero_k_bias, self.v_bias))
        qkv = torch.nn.functional.linear(x, self.mat_qkv.weight, bias).view(B, L, 3, self.num_heads, self.head_dim)
        main_type = qkv.dtype
        q, k, v = qkv.unbind(dim=2)                      # BLHc views, token stride 3 * H * c
        if self.attn_l2_norm:
            scale_mul = self.scale_mul_1H11.clamp_max(self.max_scale_mul).exp()
            oup = kv.step_normalised(q, k, v, scale_mul, self.scale, out_dtype=main_type)
        else:
            oup = kv.step(q, k, v, self.scale, out_dtype=main_type)
        return self.proj_drop(self.proj(oup.view(B, L, C)))

    attn.kv_caching = types.MethodType(kv_caching, attn)
    attn.forward = types.MethodType(forward, attn)
    return attn
