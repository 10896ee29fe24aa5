"""CPU oracle for the VAR-Q KV-cache quantization path.  TEST INFRASTRUCTURE ONLY.

This module restates, with plain torch CPU ops, the arithmetic of the reference
quantizer so that the CUDA library can be checked against it.  It is never on the
product path: only the test-suite, the smoke check and the CPU-baseline leg of the
benchmark import it.

Parity status
-------------
* Symmetric modes (the six ``G_*`` groupings, 2/4/8 bits, both layouts, multi-step
  append) are PINNED: ``tests/golden/`` holds outputs of the reference itself
  (``VAR_Q/quant.py``, ``VAR_Q/pack_unpack.py``) and ``tests/test_oracle_golden.py``
  checks this file against them bit for bit.
* Asymmetric (zero-point), ``group_size < head_dim`` and ``reduce_batch=False`` are
  extensions the reference does not implement: PARITY UNPINNED for those; this file
  is their specification.  With ``symmetric=True, group_size=None,
  reduce_batch=True`` every function below is bit-identical to the reference.
* Attention: the reference delegates to third-party kernels and pins nothing; the
  oracle is fp32 ``softmax(q k^T * scale) v`` over the dequantised cache.

Reference lines followed (paths inside the reference project):
  VAR_Q/quant.py:78-95     which dims each grouping mode reduces over
  VAR_Q/quant.py:112-116   scale = amax|x| / bound_max, clamp_min(eps)
  VAR_Q/quant.py:118-121   q = round(x / scale).clamp(bmin, bmax) -> int8
  VAR_Q/quant.py:123-124   dequant = q.float() * scale
  VAR_Q/quant.py:140-177   quant(): per-step modes vs whole-cache re-quantisation
  VAR_Q/quant.py:180-205   cache(): append / replace, scale expanded along L
  VAR_Q/quant.py:208-230   dequant_current / dequant_all / use_var_q
  VAR_Q/pack_unpack.py:167-196  little-endian bit-field packing into int32 words
  VAR_Q/pack_unpack.py:198-211  unpacking with sign extension
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

MODES = ("G_TENSOR", "G_SCALE_HEAD_DIM", "G_HEAD_DIM", "G_SCALE", "G_TOKEN", "G_TOKEN_HEAD")
PER_STEP_MODES = ("G_SCALE_HEAD_DIM", "G_SCALE", "G_TOKEN", "G_TOKEN_HEAD")
REQUANT_MODES = ("G_HEAD_DIM", "G_TENSOR")
FORMATS = ("BLHc", "BHLc")


def token_dim(fmt: str) -> int:
    """Index of the token axis L (VAR_Q/quant.py:75-76, 86)."""
    return 1 if fmt == "BLHc" else 2


def head_dim_index(fmt: str) -> int:
    return 2 if fmt == "BLHc" else 1


def reduce_dims(fmt: str, mode: str) -> Tuple[int, ...]:
    """Dims the statistics are reduced over (VAR_Q/quant.py:78-95).

    The batch dim 0 is part of every mode: scales are shared between samples.
    """
    L, H = token_dim(fmt), head_dim_index(fmt)
    if mode in ("G_TENSOR", "G_SCALE"):
        return (0, 1, 2, 3)
    if mode in ("G_SCALE_HEAD_DIM", "G_HEAD_DIM"):
        return (0, L)
    if mode == "G_TOKEN":
        return (0, H, 3)
    if mode == "G_TOKEN_HEAD":
        return (0, 3)
    raise ValueError(f"unknown grouping mode {mode}")


def bounds(bits: int) -> Tuple[int, int]:
    """Signed code range (VAR_Q/quant.py:97-98)."""
    return -(1 << (bits - 1)), (1 << (bits - 1)) - 1


# --------------------------------------------------------------------------- packing
def pack_words(codes: torch.Tensor, bits: int) -> Tuple[torch.Tensor, Dict[str, int]]:
    """int8 [..., c] -> int32 [..., ceil(c / (32/bits))]  (VAR_Q/pack_unpack.py:177-196).

    Value j of a word sits in bits [j*bits, (j+1)*bits), two's complement truncated to
    ``bits``; the tail of the last word is zero.
    """
    if bits not in (2, 4, 8):
        raise ValueError("packing is defined for 2, 4 and 8 bits")
    per = 32 // bits
    c = codes.shape[-1]
    n_words = (c + per - 1) // per
    pad = n_words * per - c
    u = codes.to(torch.int64) & ((1 << bits) - 1)
    if pad:
        u = torch.nn.functional.pad(u, (0, pad))
    u = u.reshape(*codes.shape[:-1], n_words, per)
    weights = torch.tensor([1 << (j * bits) for j in range(per)], dtype=torch.int64)
    w = (u * weights).sum(dim=-1)                 # 0 .. 2^32-1
    w = torch.where(w >= (1 << 31), w - (1 << 32), w).to(torch.int32)
    meta = {"orig_c": int(c), "vals_per_word": int(per), "pad_len": int(pad), "bits": int(bits)}
    return w, meta


def unpack_words(words: torch.Tensor, meta: Dict[str, int]) -> torch.Tensor:
    """Inverse of :func:`pack_words` with sign extension (VAR_Q/pack_unpack.py:198-211)."""
    bits, per, c = int(meta["bits"]), int(meta["vals_per_word"]), int(meta["orig_c"])
    w = words.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(per, dtype=torch.int64) * bits
    u = (w.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)
    u = u.reshape(*words.shape[:-1], words.shape[-1] * per)[..., :c]
    s = torch.where(u >= (1 << (bits - 1)), u - (1 << bits), u)
    return s.to(torch.int8)


# --------------------------------------------------------------------------- quantizer
def _stat_view(x32: torch.Tensor, fmt: str, mode: str, group_size: Optional[int], reduce_batch: bool):
    """Return (tensor to reduce, dims to reduce).  Groups along c add a 5th axis."""
    dims = reduce_dims(fmt, mode)
    if not reduce_batch:
        dims = tuple(d for d in dims if d != 0)
    c = x32.shape[-1]
    if group_size is not None and group_size != c:
        if mode != "G_TOKEN_HEAD":
            raise ValueError("group_size < head_dim is defined for G_TOKEN_HEAD only")
        if c % group_size:
            raise ValueError("head_dim must be a multiple of group_size")
        xg = x32.unflatten(-1, (c // group_size, group_size))
        dims = tuple(d for d in dims if d != 3) + (4,)
        return xg, dims, True
    return x32, dims, False


def compute_qparams(x: torch.Tensor, fmt: str, mode: str, bits: int, *, symmetric: bool = True,
                    group_size: Optional[int] = None, reduce_batch: bool = True,
                    eps: float = 1e-12) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Scale (and zero-point) of one tensor.

    Symmetric: ``scale = (amax|x| / float(bmax)).clamp_min(eps)`` (VAR_Q/quant.py:112-116).
    Asymmetric (extension): ``scale = ((max - min) / float(2^bits - 1)).clamp_min(eps)``,
    ``zp = round(bmin - min / scale)`` held as fp32 with ``-0.0`` folded to ``+0.0``.
    Shapes keep 1 in reduced dims; with groups along c the last dim is ``c / group_size``.
    """
    bmin, bmax = bounds(bits)
    x32 = x.to(torch.float32)
    xs, dims, grouped = _stat_view(x32, fmt, mode, group_size, reduce_batch)
    if symmetric:
        scale = (xs.abs().amax(dim=dims, keepdim=True) / float(bmax)).clamp_min(eps)
        zp = None
    else:
        mn = xs.amin(dim=dims, keepdim=True)
        mx = xs.amax(dim=dims, keepdim=True)
        scale = ((mx - mn) / float((1 << bits) - 1)).clamp_min(eps)
        zp = torch.round(float(bmin) - mn / scale) + 0.0
    if grouped:
        scale = scale.squeeze(-1)
        zp = None if zp is None else zp.squeeze(-1)
    return scale, zp


def _per_element(p: torch.Tensor, c: int) -> torch.Tensor:
    """Broadcastable-to-element view of a parameter whose last dim is 1, c or c/g."""
    n = p.shape[-1]
    if n in (1, c):
        return p
    return p.repeat_interleave(c // n, dim=-1)


def quantize(x: torch.Tensor, scale: torch.Tensor, zp: Optional[torch.Tensor], bits: int) -> torch.Tensor:
    """``round(x / scale) (+ zp)`` clamped to the signed range (VAR_Q/quant.py:118-121).

    True fp32 division, round-half-to-even, clamp after the round.
    """
    bmin, bmax = bounds(bits)
    x32 = x.to(torch.float32)
    c = x32.shape[-1]
    r = torch.round(x32 / _per_element(scale, c))
    if zp is not None:
        r = r + _per_element(zp, c)
    return r.clamp(bmin, bmax).to(torch.int8)


def dequantize(codes: torch.Tensor, scale: torch.Tensor, zp: Optional[torch.Tensor]) -> torch.Tensor:
    """``q.float() * scale`` (VAR_Q/quant.py:123-124); asymmetric: ``(q - zp) * scale``."""
    c = codes.shape[-1]
    q = codes.to(torch.float32)
    if zp is not None:
        q = q - _per_element(zp, c)
    return q * _per_element(scale, c)


class OracleVARQ:
    """Stateful restatement of the reference class (VAR_Q/quant.py:52-230).

    ``g_tensor_append_defect=True`` reproduces the reference's ``G_TENSOR`` behaviour of
    appending the already re-quantised cache to itself (VAR_Q/quant.py:196-201), which
    duplicates tokens; ``False`` gives the replace semantics of ``G_HEAD_DIM``
    (VAR_Q/quant.py:202-203), which is what the CUDA library implements.
    """

    def __init__(self, quant_bits=8, qkv_format="BLHc", quant_method="G_SCALE_HEAD_DIM", *,
                 symmetric=True, group_size=None, reduce_batch=True, eps=1e-12,
                 g_tensor_append_defect=False):
        assert qkv_format in FORMATS and quant_method in MODES and 1 < quant_bits <= 8
        self.bits, self.fmt, self.mode = quant_bits, qkv_format, quant_method
        self.symmetric, self.group_size, self.reduce_batch, self.eps = symmetric, group_size, reduce_batch, eps
        self.defect = g_tensor_append_defect
        self.cached_item = self.cached_scale = self.cached_zp = None
        self.quantized_item = self.scale = self.zp = None
        self.meta = None

    # VAR_Q/quant.py:180-188
    def _along_tokens(self, p, n_tokens):
        if p is None:
            return None
        d = token_dim(self.fmt)
        if p.size(d) == 1 and n_tokens > 1:
            shape = [-1] * 4
            shape[d] = n_tokens
            p = p.expand(*shape)
        return p

    def _qp(self, x):
        return compute_qparams(x, self.fmt, self.mode, self.bits, symmetric=self.symmetric,
                               group_size=self.group_size, reduce_batch=self.reduce_batch, eps=self.eps)

    # VAR_Q/quant.py:140-177
    def quant(self, item):
        if self.mode in REQUANT_MODES and self.cached_item is not None:
            item = torch.cat([self.dequant_all(), item.to(torch.float32)], dim=token_dim(self.fmt))
        scale, zp = self._qp(item)
        codes = quantize(item, scale, zp, self.bits)
        self.quantized_item, self.meta = pack_words(codes, self.bits)
        self.scale, self.zp = scale, zp

    # VAR_Q/quant.py:191-205
    def cache(self):
        n = self.quantized_item.size(token_dim(self.fmt))
        s, z = self._along_tokens(self.scale, n), self._along_tokens(self.zp, n)
        append = self.mode in PER_STEP_MODES or (self.mode == "G_TENSOR" and self.defect)
        if append and self.cached_item is not None:
            d = token_dim(self.fmt)
            self.cached_item = torch.cat([self.cached_item, self.quantized_item], dim=d)
            self.cached_scale = torch.cat([self.cached_scale, s], dim=d)
            if z is not None:
                self.cached_zp = torch.cat([self.cached_zp, z], dim=d)
        else:
            self.cached_item, self.cached_scale, self.cached_zp = self.quantized_item, s, z

    # VAR_Q/quant.py:208-224
    def dequant_current(self):
        return dequantize(unpack_words(self.quantized_item, self.meta), self.scale, self.zp)

    def dequant_all(self):
        if self.cached_item is None:
            return self.dequant_current()
        return dequantize(unpack_words(self.cached_item, self.meta), self.cached_scale, self.cached_zp)

    # VAR_Q/quant.py:227-230
    def use_var_q(self, item):
        self.quant(item)
        self.cache()
        return self.dequant_all()


# --------------------------------------------------------------------------- attention
def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, fmt: str, softmax_scale: float) -> torch.Tensor:
    """fp32 ``softmax(q k^T * scale) v`` with no mask, in the tensors' own layout.

    Stands in for the attention consumer at VAR/models/basic_var.py:156-162 and
    Infinity/infinity/models/basic.py:339-351 (non-causal at inference).
    """
    q, k, v = q.to(torch.float32), k.to(torch.float32), v.to(torch.float32)
    if fmt == "BLHc":
        q, k, v = (t.transpose(1, 2) for t in (q, k, v))
    s = torch.matmul(q, k.transpose(-1, -2)) * float(softmax_scale)
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, v)
    return o.transpose(1, 2).contiguous() if fmt == "BLHc" else o


def synthetic_kv(shape, fmt: str, seed: int, n_outlier: int = 4, outlier_gain: float = 20.0,
                 dtype=torch.float32) -> torch.Tensor:
    """Seeded N(0,1) tensor with ``n_outlier`` channels of the last dim scaled up.

    Stands in for real K/V activations, which show a few large-magnitude channels.
    """
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g, dtype=torch.float32)
    c = shape[-1]
    if n_outlier:
        idx = torch.randperm(c, generator=g)[:n_outlier]
        x[..., idx] *= outlier_gain
    return x.to(dtype)
