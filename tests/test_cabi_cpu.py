"""Host-side checks that need no GPU: the library loads, exports what the header declares,
rejects bad arguments with an error code and message, and the wrapper refuses CPU tensors."""
import ctypes
import os
import re

import pytest
import torch

from VAR_Q import _cabi
from VAR_Q.quant import VAR_Q

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _built():
    if not os.path.exists(_cabi.LIB_PATH):
        import importlib.util
        spec = importlib.util.spec_from_file_location("varq_build", os.path.join(ROOT, "var-q_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build_library()
    return _cabi.lib()


def test_library_exports_every_declared_symbol():
    lib = _built()
    header = open(os.path.join(ROOT, "include", "varq_b200.h")).read()
    declared = set(re.findall(r"\b(varq_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in the header"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/varq_b200.h but not exported"
    assert declared == set(_cabi.SYMBOLS) | {s for s in declared if s not in _cabi.SYMBOLS}
    assert lib.varq_version().startswith(b"varq_b200")


def test_argument_errors_return_codes_not_crashes():
    lib = _built()
    assert lib.varq_pack_int8(None, 4, 16, 3, None, None) == _cabi.ERR_ARG
    assert b"bits" in lib.varq_last_error()
    assert lib.varq_pack_int8(None, 4, 16, 4, None, None) == _cabi.ERR_ARG      # null pointers
    assert lib.varq_pack_int8(None, 0, 16, 4, None, None) == _cabi.OK           # empty input is fine
    t = _cabi.Tensor(None, 0, 0, 0, 0, 0)
    p = _cabi.QParams(None, None, None, 0, 0, 0, 1, 1, 0, 0, 64)
    assert lib.varq_quant_pack(t, 2, 3, 4, 64, 9, 8, 1e-12, t, p, None, 0, None) == _cabi.ERR_ARG
    assert lib.varq_quant_pack(t, 2, 3, 4, 64, 8, 4, 1e-12, t, p, None, 0, None) == _cabi.ERR_ARG   # 8-bit codes in 4-bit fields
    assert lib.varq_quant_pack(t, 2, 3, 4, 64, 4, 4, 1e-12, t, p, None, 0, None) == _cabi.ERR_ARG   # null data pointers
    assert lib.varq_quant_pack(None, 2, 3, 4, 64, 4, 4, 1e-12, t, p, None, 0, None) == _cabi.ERR_ARG
    assert lib.varq_attn_fwd(t, t, t, p, p, 1, 1, 1, 0, 64, 8, 8, 1.0, t, None, 0, None) == _cabi.ERR_ARG
    with pytest.raises(ValueError):
        _cabi.check(_cabi.ERR_ARG)


def test_workspace_queries_are_pure_host_code():
    lib = _built()
    per_dim = _cabi.QParams(None, None, None, 0, 0, 0, 1, 1, 1, 0, 1)
    assert lib.varq_quant_workspace_bytes(64, 256, 16, 64, 0, 8, per_dim) == 16 * 64 * 8
    per_tensor = _cabi.QParams(None, None, None, 0, 0, 0, 1, 1, 1, 1, 64)
    assert lib.varq_quant_workspace_bytes(64, 256, 16, 64, 0, 8, per_tensor) == 8
    assert lib.varq_attn_workspace_bytes(0, 16, 1, 100, 64, 8, 8) == 0


def test_constructor_contract_matches_reference():
    q = VAR_Q(quant_bits=4, qkv_format='BHLc', quant_method='G_TOKEN_HEAD', blk_idx=3)
    assert (q.bound_min, q.bound_max, q.cur_blk_idx, q.dim_cat) == (-8, 7, 3, 2)
    assert q.dim_map['G_TOKEN'] == (0, 1, 3) and q.dim_map['G_SCALE_HEAD_DIM'] == (0, 2)
    assert q.cached_item is None and q.cached_scale is None and q.quantized_item is None and q.scale is None
    q.qkv_format = 'BLHc'                   # Infinity re-assigns it after construction
    assert q.dim_cat == 1 and q.dim_map['G_TOKEN'] == (0, 2, 3)
    for bad in (dict(quant_bits=1), dict(quant_bits=9), dict(qkv_format='LBHc'), dict(quant_method='PER_DIM')):
        with pytest.raises(AssertionError):
            VAR_Q(**bad)
    with pytest.raises(ValueError):
        VAR_Q(quant_method='G_SCALE', group_size=32)
    with pytest.raises(ValueError):
        VAR_Q(quant_method='G_SCALE_HEAD_DIM', reduce_batch=False)


def test_cpu_tensors_are_refused_loudly():
    q = VAR_Q(quant_bits=8, quant_method='G_TOKEN_HEAD')
    with pytest.raises(RuntimeError, match="CUDA"):
        q.use_var_q(torch.zeros(1, 2, 3, 16))
    from VAR_Q.pack_unpack import pack_last_dim_to_int32_python
    with pytest.raises(RuntimeError, match="CUDA"):
        pack_last_dim_to_int32_python(torch.zeros(2, 8, dtype=torch.int8), 4)
