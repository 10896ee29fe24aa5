"""INT8 <-> packed-int32 conversion of quantized codes on the GPU.

Function names follow the reference module (VAR_Q/pack_unpack.py:107,136,177,198) so that
``from VAR_Q.pack_unpack import pack_last_dim_to_int32_triton`` keeps working; every name
is bound to the same CUDA implementation (``varq_pack_int8`` / ``varq_unpack_int8`` of
libvarq_b200.so).  Tensors must live on a CUDA device.

Format: value j of a word occupies bits [j*bits, (j+1)*bits), two's complement truncated
to ``bits``; ``32 // bits`` values per word; the tail of the last word is zero.
"""
from typing import Dict, Tuple

import torch

from . import _cabi

_HAS_TRITON = False   # the reference flag; this build has a single CUDA backend


def pack_last_dim_to_int32_cuda(q_int8: torch.Tensor, bits: int) -> Tuple[torch.Tensor, Dict[str, int]]:
    assert q_int8.dtype == torch.int8
    assert bits in (2, 4, 8), "bit-pack only implements 2/4/8 bits"
    _cabi.require_cuda(q_int8, "q_int8")
    x = q_int8.contiguous()
    *lead, c = x.shape
    vals = 32 // bits
    c_out = (c + vals - 1) // vals
    n_rows = x.numel() // c if c else 0
    out = torch.empty((*lead, c_out), dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        rc = _cabi.lib().varq_pack_int8(x.data_ptr(), n_rows, c, bits, out.data_ptr(), _cabi.stream_ptr(x.device))
    _cabi.check(rc)
    meta = {'orig_c': int(c), 'vals_per_word': int(vals), 'pad_len': int(c_out * vals - c), 'bits': int(bits)}
    return out, meta


def unpack_last_dim_from_int32_cuda(packed: torch.Tensor, meta: Dict[str, int]) -> torch.Tensor:
    assert packed.dtype == torch.int32
    _cabi.require_cuda(packed, "packed")
    bits, c = int(meta['bits']), int(meta['orig_c'])
    y = packed.contiguous()
    *lead, c_out = y.shape
    assert c_out == (c + 32 // bits - 1) // (32 // bits), "packed width does not match meta"
    n_rows = y.numel() // c_out if c_out else 0
    out = torch.empty((*lead, c), dtype=torch.int8, device=y.device)
    with torch.cuda.device(y.device):
        rc = _cabi.lib().varq_unpack_int8(y.data_ptr(), n_rows, c, bits, out.data_ptr(), _cabi.stream_ptr(y.device))
    _cabi.check(rc)
    return out


pack_last_dim_to_int32_triton = pack_last_dim_to_int32_python = pack_last_dim_to_int32_cuda
unpack_last_dim_from_int32_triton = unpack_last_dim_from_int32_python = unpack_last_dim_from_int32_cuda
