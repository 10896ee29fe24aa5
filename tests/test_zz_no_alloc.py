"""The allocation-free quantize entry point against the regular one, through the C ABI.

varq_quant_pack_static exists for callers that cannot call cudaMalloc and have no scratch to
lend (a serving process whose allocator owns all of HBM, plugin code that is not allowed to
allocate, loops that cannot afford an allocation's device-wide synchronisation).  It must give
bit-identical codes, scales and zero-points to varq_quant_pack, on repeated calls: the built-in
scratch keeps the previous call's contents, so the second call here uses data of much smaller
magnitude -- stale maxima would show up as wrong scales.

This file sorts last so that a run stopping at the first failure has already run every other
test; it also passes on its own in a fresh process (the first call does the per-device set-up).
"""
import pytest
import torch

from VAR_Q import _cabi

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _descs(x, codes, scale, zp, share_b, share_l, share_h, group):
    B, L, H, D = x.shape
    W = codes.shape[-1]
    xd = _cabi.tensor_desc(x.data_ptr(), _cabi.DTYPES[x.dtype], x.stride(0), x.stride(1), x.stride(2))
    cd = _cabi.tensor_desc(codes.data_ptr(), 0, L * H * W, H * W, W)
    nG = D // group
    nH, nL = (1 if share_h else H), (1 if share_l else L)
    p = _cabi.QParams(scale.data_ptr(), zp.data_ptr() if zp is not None else None, None,
                      nL * nH * nG, nH * nG, nG, 1, int(share_b), int(share_l), int(share_h), group)
    return xd, cd, p


def _run(fn_name, x, bits, symmetric, grouping, ws=None):
    lib = _cabi.lib()
    B, L, H, D = x.shape
    share_b, share_l, share_h, group = grouping
    W = D // (32 // bits)
    n_par = (1 if share_b else B) * (1 if share_l else L) * (1 if share_h else H) * (D // group)
    codes = torch.full((B, L, H, W), -1, dtype=torch.int32, device=DEV)
    scale = torch.full((n_par,), float("nan"), device=DEV)
    zp = None if symmetric else torch.full((n_par,), float("nan"), device=DEV)
    xd, cd, p = _descs(x, codes, scale, zp, *grouping)
    stream = _cabi.stream_ptr(x.device)
    if fn_name == "static":
        rc = lib.varq_quant_pack_static(xd, B, L, H, D, bits, bits, 1e-12, cd, p, stream)
    else:
        need = lib.varq_quant_workspace_bytes(B, L, H, D, _cabi.DTYPES[x.dtype], bits, p)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
        rc = lib.varq_quant_pack(xd, B, L, H, D, bits, bits, 1e-12, cd, p, ws.data_ptr(), need, stream)
    _cabi.check(rc)
    torch.cuda.synchronize()
    return codes, scale, zp


GROUPINGS = {
    "per_dim": (1, 1, 0, 1),          # G_SCALE_HEAD_DIM: statistics table of H*D groups
    "per_token": (1, 0, 1, 64),       # G_TOKEN: L groups
    "per_tensor": (1, 1, 1, 64),      # G_SCALE: one group
}


@pytest.mark.parametrize("name", sorted(GROUPINGS))
@pytest.mark.parametrize("symmetric", [True, False])
def test_static_scratch_matches_workspace_variant_twice(name, symmetric):
    g = torch.Generator(device=DEV).manual_seed(5)
    big = torch.randn((6, 37, 4, 64), generator=g, device=DEV) * 50.0
    small = torch.randn((6, 37, 4, 64), generator=g, device=DEV) * 0.01      # second call: far smaller range
    for call, x in enumerate((big, small)):
        want = _run("workspace", x, 4, symmetric, GROUPINGS[name])
        got = _run("static", x, 4, symmetric, GROUPINGS[name])
        for a, b, what in zip(got, want, ("codes", "scale", "zero-point")):
            if a is None:
                assert b is None
                continue
            same = torch.equal(a.view(torch.int32), b.view(torch.int32))
            assert same, f"{what} differ on call {call} ({name}, symmetric={symmetric})"


def test_static_scratch_rejects_oversized_groupings_and_reports_its_size():
    lib = _cabi.lib()
    assert lib.varq_quant_static_scratch_bytes() == 65536 * 8
    x = torch.zeros((1, 4096, 32, 64), device=DEV)
    codes = torch.empty((1, 4096, 32, 16), dtype=torch.int32, device=DEV)
    scale = torch.empty((4096 * 32,), device=DEV)
    xd, cd, p = _descs(x, codes, scale, None, 1, 0, 0, 64)      # 131072 groups > 65536
    rc = lib.varq_quant_pack_static(xd, 1, 4096, 32, 64, 8, 8, 1e-12, cd, p, _cabi.stream_ptr(x.device))
    assert rc == _cabi.ERR_WORKSPACE
    msg = lib.varq_last_error().decode()
    assert "131072" in msg and "65536" in msg
    with pytest.raises(ValueError):
        _cabi.check(rc)


def test_static_variant_makes_no_device_allocation():
    x = torch.randn((4, 16, 4, 64), device=DEV)
    _run("static", x, 8, True, GROUPINGS["per_dim"])            # set-up call for this device
    B, L, H, D = x.shape
    codes = torch.empty((B, L, H, 16), dtype=torch.int32, device=DEV)
    scale = torch.empty((H * D,), device=DEV)
    xd, cd, p = _descs(x, codes, scale, None, *GROUPINGS["per_dim"])
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        _cabi.check(_cabi.lib().varq_quant_pack_static(xd, B, L, H, D, 8, 8, 1e-12, cd, p, _cabi.stream_ptr(x.device)))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0
