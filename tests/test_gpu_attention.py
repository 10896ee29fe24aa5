"""Attention over the packed cache against the oracle: fp32 softmax(q k^T s) v on the oracle's
dequantised cache.  Tolerance (stated by the task): max-abs 2e-3 and relative L2 1e-3."""
import pytest
import torch

from oracle import varq_oracle as O
from VAR_Q.attention import attend, attend_cached
from VAR_Q.quant import VAR_Q

pytestmark = pytest.mark.gpu
DEV = "cuda"
MAX_ABS, REL_L2 = 2e-3, 1e-3


def check(out, ref, tag):
    out, ref = out.float().cpu(), ref.float().cpu()
    max_abs = (out - ref).abs().max().item()
    rel = ((out - ref).norm() / ref.norm().clamp_min(1e-30)).item()
    assert max_abs <= MAX_ABS and rel <= REL_L2, f"{tag}: max-abs {max_abs:.3e}, rel-L2 {rel:.3e}"


def build(fmt, steps, B, H, c, kq, vq, seed, q_dtype=torch.float32, k_gain=20.0):
    """Append `steps` to CUDA and oracle quantizers; returns both plus the last step's queries."""
    kd, vd = VAR_Q(qkv_format=fmt, **kq), VAR_Q(qkv_format=fmt, **vq)
    okw = lambda kw: dict(quant_bits=kw["quant_bits"], qkv_format=fmt, quant_method=kw["quant_method"],
                          **{k: v for k, v in kw.items() if k in ("symmetric", "group_size", "reduce_batch")})
    kr, vr = O.OracleVARQ(**okw(kq)), O.OracleVARQ(**okw(vq))
    for si, n in enumerate(steps):
        shape = (B, n, H, c) if fmt == "BLHc" else (B, H, n, c)
        k = O.synthetic_kv(shape, fmt, seed + 2 * si, n_outlier=4, outlier_gain=k_gain)
        v = O.synthetic_kv(shape, fmt, seed + 2 * si + 1, n_outlier=0)
        kd.append(k.to(DEV)); vd.append(v.to(DEV))
        kdeq, vdeq = kr.use_var_q(k), vr.use_var_q(v)
    g = torch.Generator().manual_seed(seed + 999)
    q = torch.randn(shape, generator=g).to(q_dtype)
    return kd, vd, kdeq, vdeq, q


def to_blhc(t, fmt):
    return t if fmt == "BLHc" else t.transpose(1, 2)


PER_HEAD8 = dict(quant_bits=8, quant_method="G_TOKEN_HEAD")
PER_DIM4A = dict(quant_bits=4, quant_method="G_SCALE_HEAD_DIM", symmetric=False)


@pytest.mark.parametrize("fmt", ["BLHc", "BHLc"])
@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("mode", O.PER_STEP_MODES)
def test_reference_modes(fmt, bits, mode):
    kq = dict(quant_bits=bits, quant_method=mode)
    scale = 0.25 / 8.0                       # VAR without l2-norm: 0.25 / sqrt(head_dim)
    kd, vd, kdeq, vdeq, q = build(fmt, (1, 4, 9, 16, 25, 36), 3, 4, 64, kq, kq, seed=bits)
    out = attend_cached(q.to(DEV), kd, vd, scale)
    ref = O.attention(q, kdeq, vdeq, fmt, scale)
    check(out, to_blhc(ref, fmt), f"{fmt} {mode} {bits}b")
    assert out.shape == (3, 36, 4, 64)


@pytest.mark.parametrize("kq,vq", [
    (PER_HEAD8, PER_HEAD8),
    (PER_DIM4A, dict(quant_bits=4, quant_method="G_TOKEN_HEAD", symmetric=False, group_size=64)),
    (dict(quant_bits=4, quant_method="G_TOKEN_HEAD", symmetric=False, group_size=32),
     dict(quant_bits=2, quant_method="G_TOKEN_HEAD", symmetric=False, group_size=32)),
    (dict(quant_bits=2, quant_method="G_TOKEN_HEAD", group_size=32, reduce_batch=False),
     dict(quant_bits=8, quant_method="G_TOKEN_HEAD", group_size=32, reduce_batch=False)),
])
@pytest.mark.parametrize("c", [64, 128])
def test_benchmark_config_quantizers(kq, vq, c):
    steps = (1, 4, 9, 16, 25, 36, 64, 100, 169, 256)          # the 256px schedule: 680 tokens
    kd, vd, kdeq, vdeq, q = build("BLHc", steps, 2, 3, c, kq, vq, seed=c)
    scale = 1.0 / (c ** 0.5)
    out = attend_cached(q.to(DEV), kd, vd, scale)
    check(out, O.attention(q, kdeq, vdeq, "BLHc", scale), f"c={c} {kq} {vq}")


@pytest.mark.parametrize("lq", [1, 2, 3, 5, 16, 37])
@pytest.mark.parametrize("q_dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_query_counts_and_dtypes_with_key_split(lq, q_dtype):
    # few (batch, head) pairs and a long cache force the split-key path and its merge kernel
    kd, vd, kdeq, vdeq, _ = build("BHLc", (700, 900, 641), 1, 2, 64, PER_HEAD8, PER_HEAD8, seed=lq)
    g = torch.Generator().manual_seed(lq)
    q = torch.randn((1, 2, lq, 64), generator=g).to(q_dtype)
    out = attend_cached(q.to(DEV), kd, vd, 0.125, out_dtype=torch.float32)
    check(out, to_blhc(O.attention(q, kdeq, vdeq, "BHLc", 0.125), "BHLc"), f"lq={lq} {q_dtype}")


def test_l2_normalised_keys_and_scaled_queries():
    # VAR with attn_l2_norm: unit-norm K, Q scaled by up to 100, softmax_scale = 1
    fmt, B, H, c = "BLHc", 2, 4, 64
    kd, vd = VAR_Q(8, fmt, "G_TOKEN_HEAD"), VAR_Q(8, fmt, "G_TOKEN_HEAD")
    kr, vr = O.OracleVARQ(8, fmt, "G_TOKEN_HEAD"), O.OracleVARQ(8, fmt, "G_TOKEN_HEAD")
    for si, n in enumerate((1, 4, 9, 16, 25, 36, 64, 100)):
        k = torch.nn.functional.normalize(O.synthetic_kv((B, n, H, c), fmt, 50 + si), dim=-1)
        v = O.synthetic_kv((B, n, H, c), fmt, 80 + si, n_outlier=0)
        qv = torch.nn.functional.normalize(O.synthetic_kv((B, n, H, c), fmt, 110 + si, n_outlier=0), dim=-1) * 12.0
        out = attend(qv.to(DEV), k.to(DEV), v.to(DEV), kd, vd, 1.0)
        ref = O.attention(qv, kr.use_var_q(k), vr.use_var_q(v), fmt, 1.0)
        check(out, ref, f"step {si}")


def test_output_dtype_and_errors():
    kd, vd, kdeq, vdeq, q = build("BLHc", (8,), 1, 2, 64, PER_HEAD8, PER_HEAD8, seed=1, q_dtype=torch.bfloat16)
    out = attend_cached(q.to(DEV), kd, vd, 0.125)
    assert out.dtype == torch.bfloat16
    ref = O.attention(q, kdeq, vdeq, "BLHc", 0.125)
    assert (out.float().cpu() - ref).abs().max() < 2e-2          # bf16 output rounding only
    with pytest.raises(ValueError):
        attend_cached(q.to(DEV), VAR_Q(8, "BLHc", "G_TOKEN_HEAD"), vd, 0.125)     # empty K cache
    with pytest.raises(ValueError):
        attend_cached(q[:, :, :1].to(DEV), kd, vd, 0.125)                         # head count mismatch
