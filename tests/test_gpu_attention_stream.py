"""The streaming small-query attention kernel (1-16 queries), forced, against the oracle.
Tolerance: max-abs 2e-3, relative L2 1e-3 (fp32 oracle on the oracle's dequantised cache)."""
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


def check(out, ref, tag):
    out, ref = out.float().cpu(), ref.float().cpu()
    max_abs = (out - ref).abs().max().item()
    rel = ((out - ref).norm() / ref.norm().clamp_min(1e-30)).item()
    assert max_abs <= 2e-3 and rel <= 1e-3, f"{tag}: max-abs {max_abs:.3e}, rel-L2 {rel:.3e}"


def make(fmt, B, H, steps, D, kb, vb, seed, mode="G_TOKEN_HEAD", **ext):
    kq, vq = VAR_Q(kb, fmt, mode, **ext), VAR_Q(vb, fmt, mode, **ext)
    kr, vr = O.OracleVARQ(kb, fmt, mode, **ext), O.OracleVARQ(vb, fmt, mode, **ext)
    for si, n in enumerate(steps):
        shape = (B, n, H, D) if fmt == "BLHc" else (B, H, n, D)
        k = O.synthetic_kv(shape, fmt, seed + 2 * si, n_outlier=4)
        v = O.synthetic_kv(shape, fmt, seed + 2 * si + 1, n_outlier=0)
        kq.append(k.to(DEV)); vq.append(v.to(DEV))
        kd, vd = kr.use_var_q(k), vr.use_var_q(v)
    return kq, vq, kd, vd


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("kb,vb", [(8, 8), (4, 4), (2, 2), (4, 2), (2, 8)])
@pytest.mark.parametrize("symmetric", [True, False])
@pytest.mark.parametrize("lq", [1, 2, 4, 7, 16])
def test_bit_widths_and_query_counts(D, kb, vb, symmetric, lq):
    kq, vq, kd, vd = make("BHLc", 2, 3, (1, 4, 9, 16, 300, 777), D, kb, vb, seed=kb + vb + lq, symmetric=symmetric)
    q = torch.randn((2, 3, lq, D), generator=torch.Generator().manual_seed(lq + D))
    _cabi.force_attn_path("stream")
    n0 = _cabi.lib().varq_launch_count()
    out = attend_cached(q.to(DEV), kq, vq, 1.0 / D ** 0.5, out_dtype=torch.float32)
    assert _cabi.lib().varq_launch_count() - n0 == 2          # few (sample, head) pairs: split over keys + merge
    check(out, O.attention(q, kd, vd, "BHLc", 1.0 / D ** 0.5).transpose(1, 2), f"D={D} k{kb} v{vb} sym={symmetric} lq={lq}")
    _cabi.force_attn_path("small")
    old = attend_cached(q.to(DEV), kq, vq, 1.0 / D ** 0.5, out_dtype=torch.float32)
    check(out, old, "stream vs small")


@pytest.mark.parametrize("mode", ["G_TOKEN", "G_SCALE"])
@pytest.mark.parametrize("lk", [1, 5, 31, 32, 33, 127, 129, 1000])
def test_ragged_cache_lengths_other_modes_and_dtypes(mode, lk):
    for q_dtype, fmt in ((torch.bfloat16, "BLHc"), (torch.float16, "BHLc")):
        kq, vq, kd, vd = make(fmt, 3, 2, (lk,), 64, 8, 4, seed=lk, mode=mode)
        shape = (3, 3, 2, 64) if fmt == "BLHc" else (3, 2, 3, 64)
        q = torch.randn(shape, generator=torch.Generator().manual_seed(lk)).to(q_dtype)
        _cabi.force_attn_path("stream")
        out = attend_cached(q.to(DEV), kq, vq, 0.125, out_dtype=torch.float32)
        ref = O.attention(q, kd, vd, fmt, 0.125)
        check(out, ref if fmt == "BLHc" else ref.transpose(1, 2), f"{mode} lk={lk} {q_dtype}")


def test_many_heads_single_launch_and_default_dispatch():
    kq, vq, kd, vd = make("BLHc", 64, 16, (40,), 64, 8, 8, seed=9)
    q = torch.randn((64, 4, 16, 64), generator=torch.Generator().manual_seed(1))
    _cabi.force_attn_path(None)
    n0 = _cabi.lib().varq_launch_count()
    out = attend_cached(q.to(DEV), kq, vq, 0.125, out_dtype=torch.float32)
    assert _cabi.lib().varq_launch_count() - n0 == 1          # enough (sample, head) pairs: no key split
    check(out, O.attention(q, kd, vd, "BLHc", 0.125), "default dispatch")


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("group", [16, 32, 64])
@pytest.mark.parametrize("kb,vb", [(8, 8), (4, 2)])
def test_groups_along_head_dim(D, group, kb, vb):
    """Asymmetric groups of 16 / 32 / 64 along head_dim: every lane applies its own group's scale and zero-point."""
    ext = dict(symmetric=False, group_size=group)
    kq, vq, kd, vd = make("BHLc", 2, 3, (1, 4, 16, 300, 500), D, kb, vb, seed=group + kb, **ext)
    for lq in (1, 5, 16):
        q = torch.randn((2, 3, lq, D), generator=torch.Generator().manual_seed(lq + D + group))
        _cabi.force_attn_path("stream")
        out = attend_cached(q.to(DEV), kq, vq, 1.0 / D ** 0.5, out_dtype=torch.float32)
        check(out, O.attention(q, kd, vd, "BHLc", 1.0 / D ** 0.5).transpose(1, 2), f"D={D} g={group} k{kb} v{vb} lq={lq}")
        _cabi.force_attn_path("small")
        check(out, attend_cached(q.to(DEV), kq, vq, 1.0 / D ** 0.5, out_dtype=torch.float32), "stream vs small")
