"""``VAR_Q`` -- KV-cache quantizer with the reference's Python API, running on B200 kernels.

Same constructor, methods and readable attributes as the reference class
(VAR_Q/quant.py:52-230), so the VAR and Infinity attention hooks
(VAR/models/basic_var.py:104-117,143-147; Infinity/infinity/models/basic.py:254-271,327-330)
work unchanged.  What differs is underneath:

* ``quant`` is one fused kernel launch (statistics, scale / zero-point, rounding, packing)
  that writes straight into a pre-allocated packed cache; there is no ``torch.cat`` growth.
* the cache is held head-major ``[B, H, L, words]`` with compact parameter tables
  (one row per token, or one row per appended step for the modes whose parameters are
  constant over a step) instead of scales materialised along L;
  ``cached_item`` / ``cached_scale`` rebuild the reference's views on demand.
* ``VAR_Q.attention.attend`` consumes the packed cache directly, so the fp32
  ``dequant_all`` round trip is only taken by callers that ask for it.

Extensions (keyword-only, defaults reproduce the reference bit for bit):
``symmetric=False`` (zero-point), ``group_size`` (groups along head_dim for
``G_TOKEN_HEAD``), ``reduce_batch=False`` (per-sample statistics), ``max_tokens``
(capacity hint).

Known deviations, both deliberate: ``G_TENSOR`` replaces the cache after re-quantising it
(the reference appends the re-quantised cache to itself, VAR_Q/quant.py:196-201, which
duplicates tokens); ``qkv_format`` may be re-assigned after construction and takes effect
(in the reference the derived dims go stale, VAR_Q/quant.py:75-95).
"""
from typing import Dict, Optional, Tuple

import torch

from . import _cabi

_METHODS = ('G_TENSOR', 'G_SCALE_HEAD_DIM', 'G_HEAD_DIM', 'G_SCALE', 'G_TOKEN', 'G_TOKEN_HEAD')
_REQUANT = ('G_HEAD_DIM', 'G_TENSOR')
# method -> (share_l, share_h, per_dim)
_GROUPING = {
    'G_TENSOR': (True, True, False), 'G_SCALE': (True, True, False),
    'G_SCALE_HEAD_DIM': (True, False, True), 'G_HEAD_DIM': (True, False, True),
    'G_TOKEN': (False, True, False), 'G_TOKEN_HEAD': (False, False, False),
}


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class VAR_Q:
    def __init__(
        self,
        quant_bits: int = 8,
        qkv_format: str = 'BLHc',
        quant_method: str = 'G_SCALE_HEAD_DIM',
        blk_idx: int = 0,
        pack_to_int32: bool = True,
        eps: float = 1e-12,
        debug: bool = False,
        *,
        symmetric: bool = True,
        group_size: Optional[int] = None,
        reduce_batch: bool = True,
        max_tokens: Optional[int] = None,
    ):
        assert qkv_format in ('BLHc', 'BHLc'), f"Invalid qkv_format: {qkv_format}"
        assert quant_method in _METHODS, f"Invalid quant_method: {quant_method}"
        assert 1 < quant_bits <= 8, "Only support (2..8] bits (common 2/4/8 bits); bit-pack implementation covers 2/4/8 bits"
        if group_size is not None and quant_method != 'G_TOKEN_HEAD':
            raise ValueError("[VAR-Q]: group_size is defined for quant_method='G_TOKEN_HEAD' only")
        if not reduce_batch and quant_method not in ('G_TOKEN', 'G_TOKEN_HEAD'):
            raise ValueError("[VAR-Q]: reduce_batch=False is defined for G_TOKEN and G_TOKEN_HEAD only")
        self.quant_bits = int(quant_bits)
        self.quant_method = quant_method
        self.cur_blk_idx = blk_idx
        self.pack_to_int32 = pack_to_int32
        self.eps = eps
        self.debug = debug
        self.symmetric = bool(symmetric)
        self.group_size = group_size
        self.reduce_batch = bool(reduce_batch)
        self.bound_min = -(2 ** (quant_bits - 1))
        self.bound_max = (2 ** (quant_bits - 1)) - 1
        self.qkv_format = qkv_format          # property: derives dim_cat / dim_map
        self._pack_meta: Optional[Dict[str, int]] = None
        self._max_tokens = max_tokens
        # device state, allocated at the first quant()
        self._codes = self._codes_next = None   # int32 [B, H, Lcap, W]
        self._scale_tbl = self._zp_tbl = None   # fp32 [nB, nH, Rcap, nG]
        self._scale_next = self._zp_next = None
        self._row_of_token = None               # int32 [Lcap] (per-step tables only)
        self._row_begin = None                  # int32 [Rcap + 1]: first token of every row (per-step tables only)
        self._shape = None                      # (B, H, D)
        self._n_tokens = self._n_rows = 0       # committed by cache()
        self._pending = None                    # (tokens, rows, replaces_cache)
        self._last = None                       # (tokens, rows) of the step committed last

    # ------------------------------------------------------------------ layout
    @property
    def qkv_format(self) -> str:
        return self._fmt

    @qkv_format.setter
    def qkv_format(self, fmt: str):
        assert fmt in ('BLHc', 'BHLc'), f"Invalid qkv_format: {fmt}"
        self._fmt = fmt
        L, H = (1, 2) if fmt == 'BLHc' else (2, 1)
        self.dim_cat = L
        self.dim_map = {
            'G_TENSOR': (0, 1, 2, 3), 'G_SCALE': (0, 1, 2, 3),
            'G_SCALE_HEAD_DIM': (0, L), 'G_HEAD_DIM': (0, L),
            'G_TOKEN': (0, H, 3), 'G_TOKEN_HEAD': (0, 3),
        }

    @property
    def store_bits(self) -> int:
        return self.quant_bits if self.pack_to_int32 else 8

    def _grouping(self, D: int) -> Tuple[bool, bool, bool, int]:
        share_l, share_h, per_dim = _GROUPING[self.quant_method]
        if per_dim:
            group = 1
        elif self.group_size is not None:
            if D % self.group_size:
                raise ValueError(f"[VAR-Q]: head_dim {D} is not a multiple of group_size {self.group_size}")
            group = int(self.group_size)
        else:
            group = D
        return self.reduce_batch, share_l, share_h, group

    def _to_internal(self, t: torch.Tensor) -> torch.Tensor:
        """item layout -> [B, H, L, *] view"""
        return t.permute(0, 2, 1, 3) if self._fmt == 'BLHc' else t

    _from_internal = _to_internal   # the permutation is its own inverse

    # ------------------------------------------------------------------ allocation
    def _ensure(self, item: torch.Tensor, n_new: int, rows_new: int, B: int, H: int, D: int):
        dev = item.device
        share_b, share_l, share_h, group = self._grouping(D)
        W = -(-D // (32 // self.store_bits))
        if self._shape is None:
            self._shape = (B, H, D)
            self._words = W
            self._nB, self._nH, self._nG = (1 if share_b else B), (1 if share_h else H), D // group
            self._lcap = self._rcap = 0
        elif self._shape != (B, H, D):
            raise ValueError(f"[VAR-Q]: item shape (B,H,c)={(B, H, D)} differs from the cache's {self._shape}")
        need_l = self._n_tokens + n_new
        if self._codes is None or need_l > self._lcap or self._codes.device != dev:
            cap = max(need_l, self._max_tokens or 0, 2 * self._lcap)
            cap = _round_up(cap, 64)
            new = torch.empty((B, H, cap, W), dtype=torch.int32, device=dev)
            rot = torch.zeros((cap,), dtype=torch.int32, device=dev) if share_l else None
            if self._codes is not None and self._n_tokens:
                new[:, :, :self._n_tokens] = self._codes[:, :, :self._n_tokens]
                if rot is not None:
                    rot[:self._n_tokens] = self._row_of_token[:self._n_tokens]
            self._codes, self._row_of_token, self._lcap = new, rot, cap
            self._codes_next = None
        need_r = self._n_rows + rows_new
        if self._scale_tbl is None or need_r > self._rcap:
            cap = (64 if share_l else self._lcap)
            cap = max(cap, need_r, 2 * self._rcap)
            shape = (self._nB, self._nH, cap, self._nG)
            s = torch.empty(shape, dtype=torch.float32, device=dev)
            z = None if self.symmetric else torch.empty(shape, dtype=torch.float32, device=dev)
            if self._scale_tbl is not None and self._n_rows:
                s[:, :, :self._n_rows] = self._scale_tbl[:, :, :self._n_rows]
                if z is not None:
                    z[:, :, :self._n_rows] = self._zp_tbl[:, :, :self._n_rows]
            if share_l:
                rb = torch.zeros((cap + 1,), dtype=torch.int32, device=dev)
                if self._row_begin is not None and self._n_rows:
                    rb[:self._n_rows + 1] = self._row_begin[:self._n_rows + 1]
                self._row_begin = rb
            self._scale_tbl, self._zp_tbl, self._rcap = s, z, cap
            self._scale_next = self._zp_next = None

    # ------------------------------------------------------------------ descriptors
    def _codes_desc(self, codes: torch.Tensor, tok0: int) -> _cabi.Tensor:
        _, H, cap, W = codes.shape
        return _cabi.tensor_desc(codes.data_ptr() + tok0 * W * 4, 0, H * cap * W, W, cap * W)

    def _param_desc(self, s_tbl, z_tbl, row0: int, D: int, rot=None) -> _cabi.QParams:
        share_b, share_l, share_h, group = self._grouping(D)
        nB, nH, cap, nG = s_tbl.shape
        off = row0 * nG * 4
        return _cabi.QParams(
            s_tbl.data_ptr() + off, (z_tbl.data_ptr() + off) if z_tbl is not None else None,
            rot.data_ptr() if rot is not None else None,
            nH * cap * nG, nG, cap * nG, 1,
            int(share_b), int(share_l), int(share_h), group)

    def _item_desc(self, t: torch.Tensor) -> _cabi.Tensor:
        sb, s1, s2, sd = t.stride()
        assert sd == 1
        sl, sh = (s1, s2) if self._fmt == 'BLHc' else (s2, s1)
        return _cabi.tensor_desc(t.data_ptr(), _cabi.DTYPES[t.dtype], sb, sl, sh)

    # ------------------------------------------------------------------ kernels
    def _quantize_into(self, item: torch.Tensor, codes, s_tbl, z_tbl, tok0: int, row0: int, stats=None):
        B, H, D = self._shape
        n = item.size(self.dim_cat)
        lib = _cabi.lib()
        grouping = self._param_desc(s_tbl, z_tbl, row0, D)
        with torch.cuda.device(item.device):
            if stats is not None:      # the statistics pass already ran inside the fused producer kernel
                rc = lib.varq_quant_pack_prestats(
                    self._item_desc(item), B, n, H, D, self.quant_bits, self.store_bits, float(self.eps),
                    self._codes_desc(codes, tok0), grouping, stats.data_ptr(), stats.numel() * stats.element_size(),
                    _cabi.stream_ptr(item.device))
            else:
                ws_bytes = lib.varq_quant_workspace_bytes(B, n, H, D, _cabi.DTYPES[item.dtype], self.store_bits, grouping)
                ws = _cabi.workspace(item.device, ws_bytes) if ws_bytes else None
                rc = lib.varq_quant_pack(
                    self._item_desc(item), B, n, H, D, self.quant_bits, self.store_bits, float(self.eps),
                    self._codes_desc(codes, tok0), grouping,
                    ws.data_ptr() if ws is not None else None, ws_bytes, _cabi.stream_ptr(item.device))
        _cabi.check(rc)

    def column_grouping(self, D: int):
        """The grouping descriptor of this quantizer if its statistics are shared over batch and tokens of a step and the
        step is quantized on its own (per-dim, per-step modes) -- the case the fused producer kernel can prepare -- else None."""
        share_b, share_l, share_h, group = self._grouping(D)
        if not (share_b and share_l) or self.quant_method in _REQUANT:
            return None
        return _cabi.QParams(None, None if self.symmetric else 1, None, 0, 0, 0, 1, 1, 1, int(share_h), group)

    def _dequant(self, codes, s_tbl, z_tbl, tok0: int, n: int, row0: int, rot, out_dtype=torch.float32, out=None):
        B, H, D = self._shape
        shape = (B, n, H, D) if self._fmt == 'BLHc' else (B, H, n, D)
        if out is None:
            out = torch.empty(shape, dtype=out_dtype, device=codes.device)
        assert tuple(out.shape) == shape and out.stride(-1) == 1
        p = self._param_desc(s_tbl, z_tbl, row0, D, rot)
        if rot is None and p.share_l:
            p.stride_r = 0          # one row describes every token of the range
        elif rot is not None:
            assert row0 == 0
            p.row_of_token = rot.data_ptr() + tok0 * 4
        with torch.cuda.device(codes.device):
            rc = _cabi.lib().varq_unpack_dequant(
                self._codes_desc(codes, tok0), B, n, H, D, self.store_bits, p,
                self._item_desc(out), _cabi.stream_ptr(codes.device))
        _cabi.check(rc)
        return out

    # ------------------------------------------------------------------ reference API
    def quant(self, item: torch.Tensor, stats: Optional[torch.Tensor] = None):
        """Quantize one appended step (VAR_Q/quant.py:140-177).  `stats`: statistics table of this very tensor as left by
        ``varq_qk_norm_stats`` (see ``column_grouping``); the kernel then skips its own statistics pass."""
        _cabi.require_cuda(item, "item")
        if item.dim() != 4:
            raise ValueError(f"[VAR-Q]: item must be 4-D ({self._fmt}), got {tuple(item.shape)}")
        if item.dtype not in _cabi.DTYPES:
            item = item.to(torch.float32)
        if self.pack_to_int32:
            assert self.quant_bits in (2, 4, 8), "bit-pack only implements 2/4/8 bits"
        if item.stride(-1) != 1:
            item = item.contiguous()
        B, D = item.size(0), item.size(3)
        n, H = (item.size(1), item.size(2)) if self._fmt == 'BLHc' else (item.size(2), item.size(1))
        vpw = 32 // self.store_bits
        meta = {'orig_c': int(D), 'vals_per_word': vpw, 'pad_len': (-D) % vpw, 'bits': self.store_bits}
        if self._pack_meta is not None and self.pack_to_int32:
            assert meta == self._pack_meta, "pack meta changed between steps"
        share_l = _GROUPING[self.quant_method][0]
        if self.quant_method in _REQUANT and self._n_tokens:
            # whole-cache modes: dequantise what is cached, join the new step, re-quantise everything
            # the dequantised cache is written straight into the head of the joint buffer and the new step behind it: no
            # concatenation pass over the whole cache (the reference does dequant_all + torch.cat, VAR_Q/quant.py:149-154)
            L0 = self._n_tokens
            full = torch.empty((B, L0 + n, H, D) if self._fmt == 'BLHc' else (B, H, L0 + n, D), dtype=torch.float32, device=item.device)
            self._dequant(self._codes, self._scale_tbl, self._zp_tbl, 0, L0, 0, self._row_of_token, out=full.narrow(self.dim_cat, 0, L0))
            full.narrow(self.dim_cat, L0, n).copy_(item)
            self._ensure(full, n, 0, B, H, D)
            if self._codes_next is None:
                self._codes_next = torch.empty_like(self._codes)
            if self._scale_next is None:
                self._scale_next = torch.empty_like(self._scale_tbl)
                self._zp_next = None if self.symmetric else torch.empty_like(self._zp_tbl)
            self._quantize_into(full, self._codes_next, self._scale_next, self._zp_next, 0, 0)
            self._pending = (full.size(self.dim_cat), 1, True)
        else:
            rows = 1 if share_l else n
            self._ensure(item, n, rows, B, H, D)
            self._quantize_into(item, self._codes, self._scale_tbl, self._zp_tbl, self._n_tokens, self._n_rows, stats)
            if share_l:
                self._row_of_token[self._n_tokens:self._n_tokens + n] = self._n_rows
                self._row_begin[self._n_rows + 1:self._n_rows + 2].fill_(self._n_tokens + n)   # entry n_rows already holds n_tokens
            self._pending = (n, rows, False)
        self._pack_meta = meta

    def cache(self):
        """Commit the step quantized last (VAR_Q/quant.py:191-205)."""
        if self._pending is None:
            raise ValueError("[VAR-Q]: cache() called before quant()")
        n, rows, replace = self._pending
        if replace:
            self._codes, self._codes_next = self._codes_next, self._codes
            self._scale_tbl, self._scale_next = self._scale_next, self._scale_tbl
            self._zp_tbl, self._zp_next = self._zp_next, self._zp_tbl
            self._row_of_token[:n] = 0
            self._row_begin[1:2].fill_(n)
            self._n_tokens, self._n_rows = n, rows
        else:
            self._n_tokens += n
            self._n_rows += rows
        self._last = (n, rows)
        self._pending = None

    def _pending_range(self):
        if self._pending is None:
            raise ValueError("[VAR-Q]: no quantized item: call quant() first")
        n, rows, replace = self._pending
        if replace:
            return self._codes_next, self._scale_next, self._zp_next, 0, n, 0, rows
        return self._codes, self._scale_tbl, self._zp_tbl, self._n_tokens, n, self._n_rows, rows

    def dequant_current(self) -> torch.Tensor:
        """fp32 dequantisation of the step quantized last (VAR_Q/quant.py:208-214)."""
        if self._pending is None and self._n_tokens:
            # after cache(): the reference's `quantized_item` still names the last step
            n, rows = self._last
            return self._dequant(self._codes, self._scale_tbl, self._zp_tbl, self._n_tokens - n, n,
                                 self._n_rows - rows, None)
        codes, s, z, tok0, n, row0, rows = self._pending_range()
        return self._dequant(codes, s, z, tok0, n, row0, None)

    def dequant_all(self) -> torch.Tensor:
        """fp32 dequantisation of the whole cache (VAR_Q/quant.py:216-224)."""
        if self._n_tokens == 0:
            return self.dequant_current()
        return self._dequant(self._codes, self._scale_tbl, self._zp_tbl, 0, self._n_tokens, 0, self._row_of_token)

    def use_var_q(self, item: torch.Tensor) -> torch.Tensor:
        """quant -> cache -> dequant_all (VAR_Q/quant.py:227-230)."""
        self.quant(item)
        self.cache()
        if self.debug:
            self.__dict__.setdefault('debug_rows', []).append(self.step_statistics(item))
        return self.dequant_all()

    # ------------------------------------------------------------------ fused path
    def append(self, item: torch.Tensor, stats: Optional[torch.Tensor] = None):
        """quant + cache without materialising the dequantised cache."""
        self.quant(item, stats)
        self.cache()
        if self.debug:
            self.__dict__.setdefault('debug_rows', []).append(self.step_statistics(item))

    @property
    def n_tokens(self) -> int:
        return self._n_tokens

    def cache_descriptors(self):
        """(codes descriptor, parameter descriptor) of the committed cache, for attention."""
        B, H, D = self._shape
        p = self._param_desc(self._scale_tbl, self._zp_tbl, 0, D, self._row_of_token)
        if self._row_of_token is not None:
            p.row_begin, p.n_rows = self._row_begin.data_ptr(), self._n_rows
        return self._codes_desc(self._codes, 0), p

    # ------------------------------------------------------------------ compact cache: save / load
    def state_dict(self) -> Dict[str, object]:
        """The committed cache in its compact on-device format: packed codes ``[B, H, L, words]``, the parameter tables
        ``[nB, nH, rows, groups]`` (one row per token, or per appended step with ``row_of_token`` / ``row_begin``), and the
        settings needed to read them.  The reference keeps scales materialised along L (VAR_Q/quant.py:180-201) and has no
        serialised form; this one is about ``bits / 8`` bytes per cached element."""
        if self._pending is not None:
            raise ValueError("[VAR-Q]: commit the quantized step with cache() before saving")
        n, r = self._n_tokens, self._n_rows
        per_step = self._row_of_token is not None
        return {
            'format': 'varq_b200.cache.v1',
            'settings': dict(quant_bits=self.quant_bits, qkv_format=self._fmt, quant_method=self.quant_method,
                             pack_to_int32=self.pack_to_int32, eps=self.eps, symmetric=self.symmetric,
                             group_size=self.group_size, reduce_batch=self.reduce_batch),
            'shape': self._shape, 'n_tokens': n, 'n_rows': r, 'pack_meta': self._pack_meta, 'last': self._last,
            'codes': None if n == 0 else self._codes[:, :, :n].clone(),
            'scale': None if n == 0 else self._scale_tbl[:, :, :r].clone(),
            'zp': None if (n == 0 or self._zp_tbl is None) else self._zp_tbl[:, :, :r].clone(),
            'row_of_token': self._row_of_token[:n].clone() if (per_step and n) else None,
            'row_begin': self._row_begin[:r + 1].clone() if (per_step and n) else None,
        }

    def load_state_dict(self, state: Dict[str, object], device=None):
        """Restore a cache written by ``state_dict`` (settings must match this quantizer's)."""
        if state.get('format') != 'varq_b200.cache.v1':
            raise ValueError("[VAR-Q]: not a varq_b200 cache")
        mine = dict(quant_bits=self.quant_bits, qkv_format=self._fmt, quant_method=self.quant_method,
                    pack_to_int32=self.pack_to_int32, eps=self.eps, symmetric=self.symmetric,
                    group_size=self.group_size, reduce_batch=self.reduce_batch)
        theirs = dict(state['settings'])
        theirs['qkv_format'] = mine['qkv_format']        # the layout of the items is a property of the caller, not of the cache
        if theirs != mine:
            raise ValueError(f"[VAR-Q]: cache was written with {state['settings']}, this quantizer has {mine}")
        self._codes = self._codes_next = self._scale_tbl = self._zp_tbl = self._scale_next = self._zp_next = None
        self._row_of_token = self._row_begin = None
        self._shape, self._n_tokens, self._n_rows, self._pending = None, 0, 0, None
        self._pack_meta, self._last = state['pack_meta'], state['last']
        n, r = int(state['n_tokens']), int(state['n_rows'])
        if n == 0:
            return self
        codes = state['codes']
        dev = torch.device(device) if device is not None else codes.device
        _cabi.require_cuda(torch.empty(0, device=dev), "the cache device")
        B, H, D = state['shape']
        probe = torch.empty((B, 1, H, D) if self._fmt == 'BLHc' else (B, H, 1, D), device=dev)
        self._ensure(probe, n, r, B, H, D)               # allocates tables of at least n tokens / r rows
        self._codes[:, :, :n] = codes.to(dev)
        self._scale_tbl[:, :, :r] = state['scale'].to(dev)
        if self._zp_tbl is not None:
            self._zp_tbl[:, :, :r] = state['zp'].to(dev)
        if self._row_of_token is not None:
            self._row_of_token[:n] = state['row_of_token'].to(dev)
            self._row_begin[:r + 1] = state['row_begin'].to(dev)
        self._n_tokens, self._n_rows = n, r
        return self

    def save(self, path: str):
        torch.save({k: (v.cpu() if torch.is_tensor(v) else v) for k, v in self.state_dict().items()}, path)

    def load(self, path: str, device='cuda'):
        return self.load_state_dict(torch.load(path, map_location='cpu', weights_only=False), device=device)

    # ------------------------------------------------------------------ range / error statistics (debug=True)
    def step_statistics(self, item: torch.Tensor) -> Dict[str, float]:
        """Range and quantization error of the step quantized last against its input ``item``: the figures the reference's
        README lists as "range stats / L2 error" (README.md:11) and its code never computes (``debug`` is stored and unused,
        VAR_Q/quant.py:61,73).  Plain torch on the device; not part of the hot path."""
        deq = self.dequant_current()
        x = item.to(torch.float32)
        err = deq - x
        sc = self.scale
        return {
            'blk_idx': int(self.cur_blk_idx), 'step_tokens': int(item.size(self.dim_cat)), 'cached_tokens': int(self._n_tokens),
            'x_min': float(x.min()), 'x_max': float(x.max()), 'x_abs_mean': float(x.abs().mean()),
            'scale_min': float(sc.min()), 'scale_max': float(sc.max()),
            'rel_l2_error': float(err.norm() / x.norm().clamp_min(1e-30)), 'max_abs_error': float(err.abs().max()),
        }

    def write_statistics_csv(self, path: str):
        """Write the rows collected by ``use_var_q`` / ``append`` while ``debug=True`` as CSV."""
        import csv
        rows = getattr(self, 'debug_rows', [])
        with open(path, 'w', newline='') as f:
            if rows:
                w = csv.DictWriter(f, fieldnames=list(rows[0].keys()))
                w.writeheader()
                w.writerows(rows)

    # ------------------------------------------------------------------ reference-shaped views
    def _ref_codes(self, codes: torch.Tensor, tok0: int, n: int) -> torch.Tensor:
        v = self._from_internal(codes[:, :, tok0:tok0 + n])
        if self.pack_to_int32:
            return v
        D = self._shape[2]
        return v.contiguous().view(torch.int8)[..., :D]

    def _ref_params(self, tbl: Optional[torch.Tensor], rows: torch.Tensor) -> Optional[torch.Tensor]:
        if tbl is None:
            return None
        return self._from_internal(tbl.index_select(2, rows))

    @property
    def quantized_item(self) -> Optional[torch.Tensor]:
        if self._pending is not None:
            codes, _, _, tok0, n, _, _ = self._pending_range()
            return self._ref_codes(codes, tok0, n)
        if self._n_tokens:
            n, _ = self._last
            return self._ref_codes(self._codes, self._n_tokens - n, n)
        return None

    def _current_params(self, which: str):
        if self._pending is not None:
            _, s, z, _, _, row0, rows = self._pending_range()
        elif self._n_tokens and self._last is not None:
            s, z = self._scale_tbl, self._zp_tbl
            rows = self._last[1]
            row0 = self._n_rows - rows
        else:
            return None
        tbl = s if which == 'scale' else z
        if tbl is None:
            return None
        return self._from_internal(tbl[:, :, row0:row0 + rows])

    @property
    def scale(self) -> Optional[torch.Tensor]:
        return self._current_params('scale')

    @property
    def zero_point(self) -> Optional[torch.Tensor]:
        return self._current_params('zp')

    @property
    def cached_item(self) -> Optional[torch.Tensor]:
        if self._n_tokens == 0:
            return None
        return self._ref_codes(self._codes, 0, self._n_tokens)

    def _cached_params(self, tbl):
        if self._n_tokens == 0 or tbl is None:
            return None
        if self._row_of_token is not None:
            rows = self._row_of_token[:self._n_tokens].to(torch.int64)
            return self._ref_params(tbl, rows)
        return self._from_internal(tbl[:, :, :self._n_tokens])

    @property
    def cached_scale(self) -> Optional[torch.Tensor]:
        return self._cached_params(self._scale_tbl)

    @property
    def cached_zero_point(self) -> Optional[torch.Tensor]:
        return self._cached_params(self._zp_tbl)
