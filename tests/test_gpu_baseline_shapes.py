"""Parity against the CPU oracle at the shapes the benchmark configurations state.

The small-shape suites cover every mode; the kernels, however, branch on size (32-bit offsets in the
single-pass quantizer, word-indexed dequantisation, key-split merges, grid limits), so this file runs
the full tensors on the GPU and keeps the CPU side at seconds by handing the oracle a slice along a
dim the statistics do NOT reduce over (a token subset for per-token-per-head groups, a head subset for
per-dim groups), or few (sample, head) pairs at full cache lengths for attention.

Bars: packed codes, scales, zero-points and dequantised values bit-exact; attention within max-abs
2e-3 and relative L2 1e-3 of fp32 attention over the oracle's dequantised cache.
"""
import pytest
import torch

from oracle import varq_oracle as O
from VAR_Q import _cabi
from VAR_Q.attention import attend_cached
from VAR_Q.quant import VAR_Q

pytestmark = pytest.mark.gpu
DEV = "cuda"

VAR_D16_STEPS = (1, 4, 9, 16, 25, 36, 64, 100, 169, 256)                       # 680 tokens
VAR_D30_STEPS = (1, 4, 9, 16, 36, 81, 169, 324, 576, 1024)                     # 2240 tokens
INFINITY_STEPS = (1, 4, 16, 36, 64, 144, 256, 400, 576, 1024, 1600, 2304, 4096)  # 10521 tokens


def bits_equal(a, b):
    a, b = a.detach().cpu().contiguous(), b.detach().cpu().contiguous()
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    return torch.equal(a.view(torch.int32), b.view(torch.int32)) if a.dtype == torch.float32 else torch.equal(a, b)


def check_attn(out, ref, tag):
    out, ref = out.float().cpu(), ref.float().cpu()
    max_abs = (out - ref).abs().max().item()
    rel = ((out - ref).norm() / ref.norm().clamp_min(1e-30)).item()
    assert max_abs <= 2e-3 and rel <= 1e-3, f"{tag}: max-abs {max_abs:.3e}, rel-L2 {rel:.3e}"


@pytest.fixture(autouse=True)
def _status_clean_and_auto_path():
    yield
    _cabi.force_attn_path(None)
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0, "a kernel wait expired"


# ------------------------------------------------------------------ configuration 1, as stated
@pytest.mark.parametrize("which,seed,n_outlier", [("K", 0, 4), ("V", 1, 4)])
def test_c1_per_head_asymmetric_int4_group64(which, seed, n_outlier):
    """fp32 [B=16, H=16, L=680, D=64] (BHLc), N(0,1) with 4 of 64 channels x20, per-(token, head)
    asymmetric INT4 with groups of 64 along D: codes, scales, zero-points, dequantised tensor."""
    x = O.synthetic_kv((16, 16, 680, 64), "BHLc", seed, n_outlier=n_outlier, outlier_gain=20.0)
    kw = dict(symmetric=False, group_size=64)
    ref = O.OracleVARQ(4, "BHLc", "G_TOKEN_HEAD", **kw)
    dut = VAR_Q(4, "BHLc", "G_TOKEN_HEAD", **kw)
    want, got = ref.use_var_q(x), dut.use_var_q(x.to(DEV))
    assert bits_equal(dut.cached_item, ref.cached_item), f"{which} codes"
    assert bits_equal(dut.cached_scale, ref.cached_scale), f"{which} scales"
    assert bits_equal(dut.cached_zero_point, ref.cached_zp), f"{which} zero-points"
    assert bits_equal(got, want), f"{which} dequantised"
    # pack / unpack round trip of the codes themselves
    codes = O.unpack_words(ref.cached_item, ref.meta)
    assert int(codes.min()) == -8 and int(codes.max()) == 7           # asymmetric codes use the whole range
    assert bits_equal(O.pack_words(codes, 4)[0], dut.cached_item)


# ------------------------------------------------------------------ full-size quantize, sliced oracle
def _gpu_randn(shape, seed, dtype=torch.float32, outliers=4, gain=20.0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    x = torch.randn(shape, generator=g, device=DEV)
    if outliers:
        x[..., :outliers] *= gain
    return x.to(dtype)


def _compare_slice(dut, ref, sl_tokens=None, sl_heads=None, fmt="BLHc", tag=""):
    """Compare the cache of `dut` restricted to a token or head subset with the oracle that saw only that subset."""
    ci, cs, cz, deq = dut.cached_item, dut.cached_scale, dut.cached_zero_point, dut.dequant_all()
    ld, hd = (1, 2) if fmt == "BLHc" else (2, 1)
    def cut(t, params=False):
        if t is None:
            return None
        if sl_tokens is not None and (not params or t.size(ld) > 1):
            t = t.index_select(ld, sl_tokens.to(t.device))
        if sl_heads is not None and (not params or t.size(hd) > 1):
            t = t.index_select(hd, sl_heads.to(t.device))
        return t
    assert bits_equal(cut(ci), ref.cached_item), "codes " + tag
    assert bits_equal(cut(cs, True), ref.cached_scale), "scales " + tag
    if ref.cached_zp is not None:
        assert bits_equal(cut(cz, True), ref.cached_zp), "zero-points " + tag
    assert bits_equal(cut(deq), ref.dequant_all()), "dequantised " + tag


def test_var_d16_last_step_whole_tensor():
    """[64, 256, 16, 64] BLHc, INT8 per-(token, head) symmetric: K fp32 contiguous, V bf16 as a strided
    view of the fused QKV activation (the benchmark's own launch shapes, single-pass kernel)."""
    B, l, H, c = 64, 256, 16, 64
    k = torch.nn.functional.normalize(_gpu_randn((B, l, H, c), 1, outliers=4, gain=6.0), dim=-1)
    qkv = _gpu_randn((B, l, 3, H, c), 2, dtype=torch.bfloat16, outliers=4, gain=6.0)
    v = qkv.unbind(dim=2)[2]
    assert not v.is_contiguous()
    for x, name in ((k, "K fp32"), (v, "V bf16 strided")):
        ref, dut = O.OracleVARQ(8, "BLHc", "G_TOKEN_HEAD"), VAR_Q(8, "BLHc", "G_TOKEN_HEAD")
        ref.use_var_q(x.cpu())
        dut.append(x)
        _compare_slice(dut, ref, tag=name)


@pytest.mark.parametrize("mode,kw,bits,slice_dim", [
    ("G_TOKEN_HEAD", dict(), 8, "tokens"),                                   # single-pass, batch-shared groups
    ("G_TOKEN_HEAD", dict(symmetric=False, group_size=64), 4, "tokens"),      # configuration 3, V
    ("G_SCALE_HEAD_DIM", dict(symmetric=False), 4, "heads"),                  # configuration 3, K (two passes)
    ("G_SCALE_HEAD_DIM", dict(), 8, "heads"),                                 # the reference's shipped setting
    ("G_TOKEN", dict(), 8, "tokens"),
])
def test_var_d30_two_largest_steps(mode, kw, bits, slice_dim):
    """[128, 576 + 1024, 30, 64] fp32 BLHc: the append offset of the last step is non-zero and the input is 1 GB."""
    B, H, c = 128, 30, 64
    dut = VAR_Q(bits, "BLHc", mode, max_tokens=1600, **kw)
    ref = O.OracleVARQ(bits, "BLHc", mode, **kw)
    g = torch.Generator().manual_seed(5)
    tok_sel = {576: torch.tensor([0, 1, 287, 575]), 1024: torch.tensor([0, 511, 1000, 1023])}
    head_sel = torch.tensor([0, 17, 29]) if mode != "G_SCALE_HEAD_DIM" else torch.tensor([13])
    picked = []
    for si, l in enumerate((576, 1024)):
        x = _gpu_randn((B, l, H, c), 10 + si)
        dut.append(x)
        if slice_dim == "tokens":
            sub = x.index_select(1, tok_sel[l].to(DEV)).cpu()
            picked.append(tok_sel[l] + (0 if si == 0 else 576))
        else:
            sub = x.index_select(2, head_sel.to(DEV)).cpu()
        ref.use_var_q(sub)
        del x
    if slice_dim == "tokens":
        _compare_slice(dut, ref, sl_tokens=torch.cat(picked), tag=f"{mode} {kw}")
    else:
        _compare_slice(dut, ref, sl_heads=head_sel, tag=f"{mode} {kw}")


@pytest.mark.parametrize("mode,kw,bits,dtype,slice_dim", [
    ("G_TOKEN_HEAD", dict(symmetric=False, group_size=32), 4, torch.float32, "tokens"),     # configuration 4, K
    ("G_TOKEN_HEAD", dict(symmetric=False, group_size=32), 2, torch.bfloat16, "tokens"),    # configuration 4, V
    ("G_TOKEN_HEAD", dict(group_size=32, reduce_batch=False), 4, torch.float32, "samples"),
    ("G_SCALE_HEAD_DIM", dict(), 8, torch.float32, "heads"),
])
def test_infinity_2b_last_step(mode, kw, bits, dtype, slice_dim):
    """[16, 16, 4096, 128] BHLc appended behind 2304 cached tokens."""
    B, H, c = 16, 16, 128
    dut = VAR_Q(bits, "BHLc", mode, max_tokens=6400, **kw)
    ref = O.OracleVARQ(bits, "BHLc", mode, **kw)
    tok_sel = {2304: torch.tensor([0, 1151, 2303]), 4096: torch.tensor([0, 1, 2047, 4095])}
    head_sel, b_sel = torch.tensor([5]), torch.tensor([0, 15])
    picked = []
    for si, l in enumerate((2304, 4096)):
        x = _gpu_randn((B, H, l, c), 20 + si, dtype=dtype)
        dut.append(x)
        if slice_dim == "tokens":
            sub = x.index_select(2, tok_sel[l].to(DEV)).cpu()
            picked.append(tok_sel[l] + (0 if si == 0 else 2304))
        elif slice_dim == "heads":
            sub = x.index_select(1, head_sel.to(DEV)).cpu()
        else:
            sub = x.index_select(0, b_sel.to(DEV)).cpu()
        ref.use_var_q(sub)
        del x
    if slice_dim == "tokens":
        _compare_slice(dut, ref, sl_tokens=torch.cat(picked), fmt="BHLc", tag=f"{mode} {kw} {dtype}")
    elif slice_dim == "heads":
        _compare_slice(dut, ref, sl_heads=head_sel, fmt="BHLc", tag=f"{mode} {kw} {dtype}")
    else:
        ci, deq = dut.cached_item.index_select(0, b_sel.to(DEV)), dut.dequant_all().index_select(0, b_sel.to(DEV))
        assert bits_equal(ci, ref.cached_item) and bits_equal(deq, ref.dequant_all())
        assert bits_equal(dut.cached_scale.index_select(0, b_sel.to(DEV)), ref.cached_scale)


# ------------------------------------------------------------------ attention at full cache lengths
def _schedule_pair(fmt, B, H, D, steps, k_args, v_args, seed, q_dtype, q_gain=1.0, normalise=False):
    """Append a whole scale schedule to GPU and oracle quantizers; yields (step index, q, K deq, V deq) after each."""
    (kb, km, kkw), (vb, vm, vkw) = k_args, v_args
    kq, vq = VAR_Q(kb, fmt, km, max_tokens=sum(steps), **kkw), VAR_Q(vb, fmt, vm, max_tokens=sum(steps), **vkw)
    kr, vr = O.OracleVARQ(kb, fmt, km, **kkw), O.OracleVARQ(vb, fmt, vm, **vkw)
    for si, l in enumerate(steps):
        shape = (B, l, H, D) if fmt == "BLHc" else (B, H, l, D)
        k = O.synthetic_kv(shape, fmt, seed + 3 * si, n_outlier=4, outlier_gain=20.0)
        v = O.synthetic_kv(shape, fmt, seed + 3 * si + 1, n_outlier=0)
        q = O.synthetic_kv(shape, fmt, seed + 3 * si + 2, n_outlier=0)
        if normalise:
            k = torch.nn.functional.normalize(k, dim=-1)
            q = torch.nn.functional.normalize(q, dim=-1) * q_gain
        q = q.to(q_dtype)
        kq.append(k.to(DEV)); vq.append(v.to(DEV))
        kd, vd = kr.use_var_q(k), vr.use_var_q(v)
        yield si, l, q, kq, vq, kd, vd


def test_c3_var_d30_schedule_every_step():
    """Configuration 3 at B=1, H=2: 2240 tokens in ten steps, K per-dim asymmetric INT4, V per-(token, head)
    asymmetric INT4 (group 64 = head_dim); every step's queries attend over everything cached, so the
    streaming, general and tensor-core kernels are all taken, the last one with Lq = 1024, Lk = 2240."""
    fmt, scale = "BLHc", 0.25 / 64 ** 0.5 * 8          # the VAR attention's 0.25 / sqrt(c), x8 to sharpen the rows
    for si, l, q, kq, vq, kd, vd in _schedule_pair(fmt, 1, 2, 64, VAR_D30_STEPS, (4, "G_SCALE_HEAD_DIM", dict(symmetric=False)),
                                                   (4, "G_TOKEN_HEAD", dict(symmetric=False, group_size=64)), 100, torch.float32):
        out = attend_cached(q.to(DEV), kq, vq, scale, out_dtype=torch.float32)
        check_attn(out, O.attention(q, kd, vd, fmt, scale), f"C3 step {si} (Lq={l}, Lk={kq.n_tokens})")


def test_c3_l2_normalised_queries_and_keys_bf16_output():
    """As the VAR attention hands them over: unit-norm K, Q scaled by its learnt gain, softmax_scale 1."""
    fmt = "BLHc"
    for si, l, q, kq, vq, kd, vd in _schedule_pair(fmt, 2, 1, 64, VAR_D30_STEPS, (4, "G_SCALE_HEAD_DIM", dict(symmetric=False)),
                                                   (4, "G_TOKEN_HEAD", dict(symmetric=False, group_size=64)), 200, torch.float32,
                                                   q_gain=8.0, normalise=True):
        if l < 324:
            continue
        out = attend_cached(q.to(DEV), kq, vq, 1.0, out_dtype=torch.float32)
        check_attn(out, O.attention(q, kd, vd, fmt, 1.0), f"C3 normalised step {si}")


@pytest.mark.parametrize("q_dtype", [torch.float32, torch.bfloat16])
def test_c4_infinity_schedule(q_dtype):
    """Configuration 4 at B=1, H=2: head_dim 128, 13 steps to 10 521 tokens, K INT4 / V INT2 in asymmetric groups
    of 32; queries of 1, 4, 16 and 4096 tokens (the first three and the last step) attend over their caches,
    and a 16-query block attends over the complete cache."""
    fmt, D = "BHLc", 128
    scale = 1.0 / D ** 0.5
    last = None
    for si, l, q, kq, vq, kd, vd in _schedule_pair(fmt, 1, 2, D, INFINITY_STEPS, (4, "G_TOKEN_HEAD", dict(symmetric=False, group_size=32)),
                                                   (2, "G_TOKEN_HEAD", dict(symmetric=False, group_size=32)), 300, q_dtype):
        last = (q, kq, vq, kd, vd)
        if l not in (1, 4, 16, 4096):
            continue
        out = attend_cached(q.to(DEV), kq, vq, scale, out_dtype=torch.float32)
        check_attn(out, O.attention(q, kd, vd, fmt, scale).transpose(1, 2), f"C4 {q_dtype} step {si} (Lq={l}, Lk={kq.n_tokens})")
    q, kq, vq, kd, vd = last
    for lq in (1, 16):
        qs = q[:, :, :lq].contiguous()
        out = attend_cached(qs.to(DEV), kq, vq, scale, out_dtype=torch.float32)
        check_attn(out, O.attention(qs, kd, vd, fmt, scale).transpose(1, 2), f"C4 {q_dtype} Lq={lq} over 10 521 tokens")


_SWEEP_CACHE = {}


def _sweep_cache(D, bits, grouped):
    """One packed cache of 10 521 tokens (13 appended steps) per (head_dim, bits, grouping), shared by the query counts."""
    key = (D, bits, grouped)
    if key not in _SWEEP_CACHE:
        kw = dict(group_size=32, symmetric=False) if grouped else {}
        last = None
        for last in _schedule_pair("BHLc", 1, 2, D, INFINITY_STEPS, (bits, "G_TOKEN_HEAD", kw), (bits, "G_TOKEN_HEAD", kw),
                                   1000 + D + bits, torch.bfloat16):
            pass
        _, _, _, kq, vq, kd, vd = last
        _SWEEP_CACHE.clear()            # keep one cache alive at a time
        _SWEEP_CACHE[key] = (kq, vq, kd, vd)
    return _SWEEP_CACHE[key]


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("bits", [8, 4, 2])
@pytest.mark.parametrize("grouped", [False, True], ids=["per_head", "group32"])
@pytest.mark.parametrize("lq", [1, 16, 256, 1024, 4096])
def test_c5_sweep_grid(D, bits, grouped, lq):
    """Isolated dequant-attention sweep at B=1, H=2: bf16 N(0,1) queries against 10 521 packed tokens whose K has four
    channels x20; per-(token, head) symmetric scales and asymmetric groups of 32."""
    kq, vq, kd, vd = _sweep_cache(D, bits, grouped)
    q = O.synthetic_kv((1, 2, lq, D), "BHLc", 77 + lq, n_outlier=0, dtype=torch.bfloat16)
    scale = 1.0 / D ** 0.5
    out = attend_cached(q.to(DEV), kq, vq, scale, out_dtype=torch.float32)
    check_attn(out, O.attention(q, kd, vd, "BHLc", scale).transpose(1, 2), f"C5 D={D} {bits}b grouped={grouped} Lq={lq}")


def test_grid_limit_many_sample_head_pairs():
    """More (sample, head) pairs than one grid dimension of the tensor-core launch holds."""
    B, H, D, lk, lq = 4200, 16, 64, 40, 20           # 67 200 pairs
    g = torch.Generator(device=DEV).manual_seed(3)
    k = torch.randn((B, lk, H, D), generator=g, device=DEV)
    v = torch.randn((B, lk, H, D), generator=g, device=DEV)
    q = torch.randn((B, lq, H, D), generator=g, device=DEV)
    kq, vq = VAR_Q(8, "BLHc", "G_TOKEN_HEAD", reduce_batch=False), VAR_Q(8, "BLHc", "G_TOKEN_HEAD", reduce_batch=False)
    kq.append(k); vq.append(v)
    out = attend_cached(q, kq, vq, 0.125, out_dtype=torch.float32)
    sel = torch.tensor([0, 1, 4095, 4096, 4199])
    kr, vr = O.OracleVARQ(8, "BLHc", "G_TOKEN_HEAD", reduce_batch=False), O.OracleVARQ(8, "BLHc", "G_TOKEN_HEAD", reduce_batch=False)
    kd, vd = kr.use_var_q(k[sel.to(DEV)].cpu()), vr.use_var_q(v[sel.to(DEV)].cpu())
    check_attn(out[sel.to(DEV)], O.attention(q[sel.to(DEV)].cpu(), kd, vd, "BLHc", 0.125), "B*H > 65535")
