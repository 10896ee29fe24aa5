"""Guard words around every output buffer, through the C ABI.

A memory checker cannot be run on the GPU pool, so out-of-bounds stores are looked for directly: each
output a kernel writes (packed codes, scales, zero-points, dequantised values, attention output,
key-split partials) is carved out of a larger buffer filled with a sentinel, the call is made on ragged
shapes (head_dim not a multiple of the codes per word, cache length not a multiple of any tile, one
query), and the sentinels on both sides must survive while the payload is fully overwritten where the
contract says so.
"""
import pytest
import torch

from oracle import varq_oracle as O
from VAR_Q import _cabi
from VAR_Q.quant import VAR_Q

pytestmark = pytest.mark.gpu
DEV = "cuda"
PAD = 256            # guard elements on each side
SENTINEL_I32 = 0x5A5A5A5A


class Guarded:
    """`n` elements of `dtype` between two runs of sentinel words."""

    def __init__(self, n, dtype):
        self.dtype, self.n = dtype, n
        es = torch.empty((), dtype=dtype).element_size()
        total_bytes = (n + 2 * PAD) * es
        self.raw = torch.full(((total_bytes + 3) // 4 + 1,), SENTINEL_I32, dtype=torch.int32, device=DEV)
        self.flat = self.raw.view(torch.uint8)[: total_bytes].view(dtype)
        self.payload = self.flat[PAD: PAD + n]

    def ptr(self):
        return self.payload.data_ptr()

    def assert_intact(self, what):
        sent = torch.full((1,), SENTINEL_I32, dtype=torch.int32).view(torch.uint8)
        raw = self.raw.view(torch.uint8).cpu()
        es = self.payload.element_size()
        lo, hi = PAD * es, (PAD + self.n) * es
        want = sent.repeat(raw.numel() // 4)
        assert torch.equal(raw[:lo], want[:lo]), f"{what}: store below the buffer"
        assert torch.equal(raw[hi:], want[hi:]), f"{what}: store past the buffer"


def _quant_call(x, bits, share, group, symmetric):
    """varq_quant_pack on guarded outputs; returns (codes, scale, zp) payload views."""
    B, L, H, D = x.shape
    share_b, share_l, share_h = share
    W = -(-D // (32 // bits))
    nB, nL, nH, nG = (1 if share_b else B), (1 if share_l else L), (1 if share_h else H), D // group
    codes = Guarded(B * L * H * W, torch.int32)
    scale = Guarded(nB * nL * nH * nG, torch.float32)
    zp = None if symmetric else Guarded(nB * nL * nH * nG, torch.float32)
    lib = _cabi.lib()
    xd = _cabi.tensor_desc(x.data_ptr(), _cabi.DTYPES[x.dtype], x.stride(0), x.stride(1), x.stride(2))
    cd = _cabi.tensor_desc(codes.ptr(), 0, L * H * W, H * W, W)
    p = _cabi.QParams(scale.ptr(), zp.ptr() if zp else None, None, nL * nH * nG, nH * nG, nG, 1,
                      int(share_b), int(share_l), int(share_h), group)
    need = lib.varq_quant_workspace_bytes(B, L, H, D, _cabi.DTYPES[x.dtype], bits, p)
    ws = Guarded(max(need, 16), torch.uint8)
    _cabi.check(lib.varq_quant_pack(xd, B, L, H, D, bits, bits, 1e-12, cd, p, ws.ptr(), need, _cabi.stream_ptr(x.device)))
    torch.cuda.synchronize()
    for g, name in ((codes, "codes"), (scale, "scale"), (zp, "zero-point"), (ws, "workspace")):
        if g is not None:
            g.assert_intact(f"varq_quant_pack {name} shape={tuple(x.shape)} bits={bits} share={share} group={group}")
    assert not bool((codes.payload == SENTINEL_I32).all()), "codes were not written"
    return codes, scale, zp, p, (B, L, H, D, W)


GROUPINGS = [((1, 0, 0), None), ((0, 0, 0), None), ((1, 1, 0), 1), ((1, 1, 1), None), ((1, 0, 1), None)]


@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("share,group", GROUPINGS)
@pytest.mark.parametrize("symmetric", [True, False])
def test_quantize_and_dequantize_stay_inside_their_buffers(bits, share, group, symmetric):
    for shape, dtype in (((3, 7, 2, 20), torch.float32), ((2, 5, 3, 5), torch.bfloat16), ((8, 33, 4, 64), torch.float32),
                         ((1, 1, 1, 36), torch.float16)):
        B, L, H, D = shape
        x = O.synthetic_kv(shape, "BLHc", D + bits, n_outlier=1, dtype=dtype).to(DEV)
        codes, scale, zp, p, (B, L, H, D, W) = _quant_call(x, bits, share, group or D, symmetric)
        # dequantise the same codes into a guarded fp32 buffer, and compare with the oracle
        out = Guarded(B * L * H * D, torch.float32)
        cd = _cabi.tensor_desc(codes.ptr(), 0, L * H * W, H * W, W)
        od = _cabi.tensor_desc(out.ptr(), _cabi.F32, L * H * D, H * D, D)
        _cabi.check(_cabi.lib().varq_unpack_dequant(cd, B, L, H, D, bits, p, od, _cabi.stream_ptr(x.device)))
        torch.cuda.synchronize()
        out.assert_intact(f"varq_unpack_dequant shape={shape} bits={bits}")
        mode = {(1, 0, 0): "G_TOKEN_HEAD", (0, 0, 0): "G_TOKEN_HEAD", (1, 1, 0): "G_SCALE_HEAD_DIM", (1, 1, 1): "G_SCALE",
                (1, 0, 1): "G_TOKEN"}[share]
        ref = O.OracleVARQ(bits, "BLHc", mode, symmetric=symmetric, reduce_batch=bool(share[0]))
        want = ref.use_var_q(x.cpu())
        got = out.payload.view(B, L, H, D).cpu()
        assert torch.equal(got.view(torch.int32), want.view(torch.int32)), f"dequantised values shape={shape} bits={bits} share={share}"
        assert torch.equal(codes.payload.view(B, L, H, W).cpu(), ref.cached_item)


def test_shared_token_descriptor_with_the_producers_row_stride():
    """A consumer may hand back the descriptor it gave varq_quant_pack unchanged: with share_l = 1 and no row table
    the row stride is ignored, as the header says, whatever value it holds."""
    x = O.synthetic_kv((2, 9, 3, 32), "BLHc", 5).to(DEV)
    codes, scale, zp, p, (B, L, H, D, W) = _quant_call(x, 8, (1, 1, 0), 1, True)
    assert p.stride_r != 0 and p.share_l == 1 and not p.row_of_token
    out = Guarded(B * L * H * D, torch.float32)
    cd = _cabi.tensor_desc(codes.ptr(), 0, L * H * W, H * W, W)
    od = _cabi.tensor_desc(out.ptr(), _cabi.F32, L * H * D, H * D, D)
    _cabi.check(_cabi.lib().varq_unpack_dequant(cd, B, L, H, D, 8, p, od, _cabi.stream_ptr(x.device)))
    torch.cuda.synchronize()
    out.assert_intact("shared-token descriptor")
    ref = O.OracleVARQ(8, "BLHc", "G_SCALE_HEAD_DIM")
    want = ref.use_var_q(x.cpu())
    assert torch.equal(out.payload.view(B, L, H, D).cpu().view(torch.int32), want.view(torch.int32))


def _attn_call(path, q, kq, vq, scale, out_dtype):
    B, D = q.size(0), q.size(3)
    Lq, H = q.size(2), q.size(1)                      # q is BHLc here
    Lk = kq.n_tokens
    lib = _cabi.lib()
    out = Guarded(B * Lq * H * D, out_dtype)
    kc, kp = kq.cache_descriptors()
    vc, vp = vq.cache_descriptors()
    need = lib.varq_attn_workspace_bytes(B, H, Lq, Lk, D, kq.store_bits, vq.store_bits)
    ws = Guarded(max(need, 16), torch.uint8)
    qd = kq._item_desc(q)
    od = _cabi.tensor_desc(out.ptr(), _cabi.DTYPES[out_dtype], Lq * H * D, H * D, D)
    _cabi.force_attn_path(path)
    n0 = lib.varq_launch_count()
    _cabi.check(lib.varq_attn_fwd(qd, kc, vc, kp, vp, B, H, Lq, Lk, D, kq.store_bits, vq.store_bits, float(scale), od,
                                  ws.ptr(), need, _cabi.stream_ptr(q.device)))
    torch.cuda.synchronize()
    _cabi.force_attn_path(None)
    assert _cabi.device_status() == 0
    out.assert_intact(f"varq_attn_fwd[{path}] output Lq={Lq} Lk={Lk} D={D}")
    ws.assert_intact(f"varq_attn_fwd[{path}] workspace Lq={Lq} Lk={Lk} D={D}")
    return out.payload.view(B, Lq, H, D), lib.varq_launch_count() - n0


@pytest.mark.parametrize("path", ["small", "stream", "tc", "mid"])
@pytest.mark.parametrize("D,kb,vb", [(64, 8, 4), (128, 4, 2)])
@pytest.mark.parametrize("lq,lk", [(1, 1), (1, 333), (3, 129), (16, 2047), (17, 65), (130, 131), (257, 1000)])
def test_attention_kernels_stay_inside_their_buffers(path, D, kb, vb, lq, lk):
    fmt, B, H = "BHLc", 2, 3
    kq, vq = VAR_Q(kb, fmt, "G_TOKEN_HEAD", symmetric=False), VAR_Q(vb, fmt, "G_TOKEN_HEAD", symmetric=False)
    kr, vr = O.OracleVARQ(kb, fmt, "G_TOKEN_HEAD", symmetric=False), O.OracleVARQ(vb, fmt, "G_TOKEN_HEAD", symmetric=False)
    k = O.synthetic_kv((B, H, lk, D), fmt, lk, n_outlier=2)
    v = O.synthetic_kv((B, H, lk, D), fmt, lk + 1, n_outlier=0)
    kq.append(k.to(DEV)); vq.append(v.to(DEV))
    kd, vd = kr.use_var_q(k), vr.use_var_q(v)
    q = torch.randn((B, H, lq, D), generator=torch.Generator().manual_seed(lq))
    for out_dtype in (torch.float32, torch.bfloat16):
        out, _ = _attn_call(path, q.to(DEV), kq, vq, 1.0 / D ** 0.5, out_dtype)
        ref = O.attention(q, kd, vd, fmt, 1.0 / D ** 0.5).transpose(1, 2)
        tol = 2e-3 if out_dtype == torch.float32 else 2e-2
        assert (out.float().cpu() - ref).abs().max().item() <= tol
