"""The warp-level tensor-core kernel for the early scales (tens of queries over a few hundred cached tokens), forced
for every case, against the oracle.  Tolerance: max-abs 2e-3, relative L2 1e-3 (fp32 oracle)."""
import pytest
import torch

from oracle import varq_oracle as O
from VAR_Q import _cabi
from VAR_Q.attention import attend_cached
from VAR_Q.quant import VAR_Q

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _auto_path_afterwards():
    yield
    _cabi.force_attn_path(None)


def run(q, kq, vq, scale, out_dtype=torch.float32):
    _cabi.force_attn_path("mid")
    n0 = _cabi.lib().varq_launch_count()
    out = attend_cached(q, kq, vq, scale, out_dtype=out_dtype)
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0
    return out, _cabi.lib().varq_launch_count() - n0


def make(fmt, B, H, steps, kb, vb, seed, mode, **ext):
    D = 64
    kq, vq = VAR_Q(kb, fmt, mode, **ext), VAR_Q(vb, fmt, mode, **ext)
    kr, vr = O.OracleVARQ(kb, fmt, mode, **ext), O.OracleVARQ(vb, fmt, mode, **ext)
    for si, n in enumerate(steps):
        shape = (B, n, H, D) if fmt == "BLHc" else (B, H, n, D)
        k = O.synthetic_kv(shape, fmt, seed + 2 * si, n_outlier=4)
        v = O.synthetic_kv(shape, fmt, seed + 2 * si + 1, n_outlier=0)
        kq.append(k.to(DEV)); vq.append(v.to(DEV))
        kd, vd = kr.use_var_q(k), vr.use_var_q(v)
    return kq, vq, kd, vd


def check(out, ref, tag):
    out, ref = out.float().cpu(), ref.float().cpu()
    max_abs = (out - ref).abs().max().item()
    rel = ((out - ref).norm() / ref.norm().clamp_min(1e-30)).item()
    assert max_abs <= 2e-3 and rel <= 1e-3, f"{tag}: max-abs {max_abs:.3e}, rel-L2 {rel:.3e}"


@pytest.mark.parametrize("kb,vb", [(8, 8), (4, 4), (2, 2), (4, 2), (8, 2), (2, 8)])
@pytest.mark.parametrize("symmetric", [True, False])
@pytest.mark.parametrize("fmt", ["BLHc", "BHLc"])
def test_bit_widths_and_layouts(kb, vb, symmetric, fmt):
    steps = (1, 4, 9, 16, 25, 36, 64)                   # 155 cached tokens: two full chunks and a ragged one
    kq, vq, kd, vd = make(fmt, 2, 3, steps, kb, vb, kb * 10 + vb, "G_TOKEN_HEAD", symmetric=symmetric)
    qs = (2, 64, 3, 64) if fmt == "BLHc" else (2, 3, 64, 64)
    q = torch.randn(qs, generator=torch.Generator().manual_seed(kb + vb))
    out, launches = run(q.to(DEV), kq, vq, 0.125)
    assert launches == 1
    ref = O.attention(q, kd, vd, fmt, 0.125)
    check(out, ref if fmt == "BLHc" else ref.transpose(1, 2), f"k{kb} v{vb} sym={symmetric} {fmt}")


@pytest.mark.parametrize("lq", [5, 9, 16, 17, 25, 63, 64, 65, 100, 128])
@pytest.mark.parametrize("lk", [1, 7, 63, 64, 65, 130, 255, 384])
def test_ragged_shapes(lq, lk):
    kq, vq, kd, vd = make("BLHc", 1, 2, (lk,), 8, 4, lq + lk, "G_TOKEN_HEAD", symmetric=False)
    q = torch.randn((1, lq, 2, 64), generator=torch.Generator().manual_seed(lq * 1000 + lk))
    out, _ = run(q.to(DEV), kq, vq, 0.125)
    check(out, O.attention(q, kd, vd, "BLHc", 0.125), f"lq={lq} lk={lk}")


@pytest.mark.parametrize("q_dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("mode", ["G_TOKEN_HEAD", "G_TOKEN", "G_SCALE"])
def test_query_dtypes_and_per_key_groupings(q_dtype, mode):
    kq, vq, kd, vd = make("BLHc", 2, 4, (1, 4, 9, 16, 25, 36, 64, 100), 8, 8, 77, mode)
    q = (torch.nn.functional.normalize(torch.randn((2, 100, 4, 64), generator=torch.Generator().manual_seed(3)), dim=-1) * 4).to(q_dtype)
    for out_dtype in (torch.float32, torch.bfloat16):
        out, _ = run(q.to(DEV), kq, vq, 1.0, out_dtype)
        ref = O.attention(q.float(), kd, vd, "BLHc", 1.0)
        if out_dtype == torch.float32:
            check(out, ref, f"{mode} {q_dtype}")
        else:
            assert (out.float().cpu() - ref).abs().max().item() <= 2e-3 + 4e-3 * ref.abs().max().item()


def test_other_groupings_go_elsewhere():
    """Scales that vary along head_dim are not taken: the call falls through to another kernel and stays correct."""
    kq, vq, kd, vd = make("BLHc", 1, 2, (30, 40), 4, 4, 5, "G_TOKEN_HEAD", symmetric=False, group_size=32)
    q = torch.randn((1, 40, 2, 64), generator=torch.Generator().manual_seed(9))
    out, _ = run(q.to(DEV), kq, vq, 0.125)
    check(out, O.attention(q, kd, vd, "BLHc", 0.125), "group 32")


@pytest.mark.parametrize("gain", [1e-3, 3e4])
def test_v_scales_far_from_one(gain):
    """The V scale is folded into the softmax weights through the exponent, so the fp16 operand stays normalised for
    small and for huge V values alike (scales below 2^-20 are folded as 2^-20, like in the tcgen05 kernel); the result is
    compared relative to its own magnitude."""
    kq, vq = VAR_Q(8, "BLHc", "G_TOKEN_HEAD"), VAR_Q(8, "BLHc", "G_TOKEN_HEAD", symmetric=False)
    kr, vr = O.OracleVARQ(8, "BLHc", "G_TOKEN_HEAD"), O.OracleVARQ(8, "BLHc", "G_TOKEN_HEAD", symmetric=False)
    for si, n in enumerate((40, 60)):
        k = O.synthetic_kv((2, n, 2, 64), "BLHc", 11 + si, n_outlier=4)
        v = gain * O.synthetic_kv((2, n, 2, 64), "BLHc", 21 + si, n_outlier=0)
        kq.append(k.to(DEV)); vq.append(v.to(DEV))
        kd, vd = kr.use_var_q(k), vr.use_var_q(v)
    q = torch.randn((2, 30, 2, 64), generator=torch.Generator().manual_seed(4))
    out, _ = run(q.to(DEV), kq, vq, 0.125)
    ref = O.attention(q, kd, vd, "BLHc", 0.125)
    out = out.float().cpu()
    assert (out - ref).abs().max().item() <= 2e-3 * ref.abs().max().item()
    assert ((out - ref).norm() / ref.norm()).item() <= 1e-3
