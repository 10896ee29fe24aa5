"""The tensor-core (tcgen05/TMEM) attention kernel, forced for every case, against the oracle
and against the CUDA-core kernel.  Tolerance: max-abs 2e-3, relative L2 1e-3 (fp32 oracle)."""
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


def run(path, q, kq, vq, scale, out_dtype=torch.float32):
    _cabi.force_attn_path(path)
    n0 = _cabi.lib().varq_launch_count()
    out = attend_cached(q, kq, vq, scale, out_dtype=out_dtype)
    torch.cuda.synchronize()
    status = _cabi.device_status()
    assert status == 0, f"a kernel wait expired (code {status})"
    return out, _cabi.lib().varq_launch_count() - n0


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


def check(out, ref, tag):
    out, ref = out.float().cpu(), ref.float().cpu()
    max_abs = (out - ref).abs().max().item()
    rel = ((out - ref).norm() / ref.norm().clamp_min(1e-30)).item()
    assert max_abs <= 2e-3 and rel <= 1e-3, f"{tag}: max-abs {max_abs:.3e}, rel-L2 {rel:.3e}"


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("kb,vb", [(8, 8), (4, 4), (2, 2), (4, 2), (8, 2), (2, 8)])
@pytest.mark.parametrize("symmetric", [True, False])
def test_bit_widths(D, kb, vb, symmetric):
    kq, vq, kd, vd = make("BHLc", 2, 3, (1, 4, 9, 16, 25, 36, 64, 100, 169, 256), D, kb, vb, seed=kb * 10 + vb, symmetric=symmetric)
    q = torch.randn((2, 3, 256, D), generator=torch.Generator().manual_seed(D + kb))
    out, launches = run("tc", q.to(DEV), kq, vq, 1.0 / D ** 0.5)
    assert launches == 2          # per-key parameter preparation + the attention kernel
    check(out, O.attention(q, kd, vd, "BHLc", 1.0 / D ** 0.5).transpose(1, 2), f"D={D} k{kb} v{vb} sym={symmetric}")


@pytest.mark.parametrize("lq", [1, 9, 16, 100, 128, 129, 300])
@pytest.mark.parametrize("lk", [1, 63, 64, 65, 127, 128, 129, 700])
def test_ragged_tiles(lq, lk):
    kq, vq, kd, vd = make("BLHc", 1, 2, (lk,), 64, 8, 4, seed=lq + lk)
    q = torch.randn((1, lq, 2, 64), generator=torch.Generator().manual_seed(lq * 1000 + lk))
    out, _ = run("tc", q.to(DEV), kq, vq, 0.125)
    check(out, O.attention(q, kd, vd, "BLHc", 0.125), f"lq={lq} lk={lk}")
    kq2, vq2, kd2, vd2 = make("BLHc", 1, 2, (lk,), 128, 4, 8, seed=lq + lk + 1)
    q2 = torch.randn((1, lq, 2, 128), generator=torch.Generator().manual_seed(lq * 1000 + lk + 1))
    out2, _ = run("tc", q2.to(DEV), kq2, vq2, 0.09)
    check(out2, O.attention(q2, kd2, vd2, "BLHc", 0.09), f"D=128 lq={lq} lk={lk}")


@pytest.mark.parametrize("q_dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("mode", ["G_TOKEN_HEAD", "G_TOKEN", "G_SCALE"])
def test_query_dtypes_modes_and_agreement_with_cuda_core_kernel(q_dtype, mode):
    kq, vq, kd, vd = make("BLHc", 2, 4, (30, 500, 470), 64, 8, 8, seed=3, mode=mode)
    q = torch.randn((2, 200, 4, 64), generator=torch.Generator().manual_seed(5)).to(q_dtype)
    tc, _ = run("tc", q.to(DEV), kq, vq, 0.125)
    cc, _ = run("small", q.to(DEV), kq, vq, 0.125)
    ref = O.attention(q, kd, vd, "BLHc", 0.125)
    check(tc, ref, f"tc {mode} {q_dtype}")
    check(cc, ref, f"small {mode} {q_dtype}")
    check(tc, cc, "tc vs small")


def test_large_logits_l2_normalised_keys():
    # unit-norm K, queries scaled by 30 and 100: logits up to +-100, sharply peaked rows
    fmt, B, H, D = "BLHc", 2, 2, 64
    for gain in (30.0, 100.0):
        kq, vq = VAR_Q(8, fmt, "G_TOKEN_HEAD"), VAR_Q(8, fmt, "G_TOKEN_HEAD")
        kr, vr = O.OracleVARQ(8, fmt, "G_TOKEN_HEAD"), O.OracleVARQ(8, fmt, "G_TOKEN_HEAD")
        k = torch.nn.functional.normalize(O.synthetic_kv((B, 680, H, D), fmt, 1), dim=-1)
        v = O.synthetic_kv((B, 680, H, D), fmt, 2, n_outlier=0)
        kq.append(k.to(DEV)); vq.append(v.to(DEV))
        q = torch.nn.functional.normalize(torch.randn((B, 256, H, D), generator=torch.Generator().manual_seed(3)), dim=-1) * gain
        out, _ = run("tc", q.to(DEV), kq, vq, 1.0)
        check(out, O.attention(q, kr.use_var_q(k), vr.use_var_q(v), fmt, 1.0), f"gain {gain}")


def test_full_size_last_scale_is_linear_in_v_and_permutation_invariant():
    """VAR-d16 last scale (B2=64, H=16, Lq=256, Lk=680): too large for the CPU oracle in seconds.
    Properties: (i) tensor-core and CUDA-core kernels agree; (ii) attention is invariant to a
    permutation of the cached tokens (K and V permuted together)."""
    B, H, Lq, Lk, D = 64, 16, 256, 680, 64
    g = torch.Generator(device=DEV).manual_seed(0)
    k = torch.nn.functional.normalize(torch.randn((B, Lk, H, D), generator=g, device=DEV), dim=-1)
    v = torch.randn((B, Lk, H, D), generator=g, device=DEV)
    q = torch.nn.functional.normalize(torch.randn((B, Lq, H, D), generator=g, device=DEV), dim=-1) * 4
    def cached(kk, vv):
        # per-sample statistics: the codes of a token do not depend on its position in the cache
        a, b = VAR_Q(8, "BLHc", "G_TOKEN_HEAD", reduce_batch=False), VAR_Q(8, "BLHc", "G_TOKEN_HEAD", reduce_batch=False)
        a.append(kk); b.append(vv)
        return a, b
    kq, vq = cached(k, v)
    tc, _ = run("tc", q, kq, vq, 1.0)
    cc, _ = run("small", q, kq, vq, 1.0)
    check(tc, cc, "tc vs small at full size")
    perm = torch.randperm(Lk, generator=torch.Generator().manual_seed(1)).to(DEV)
    kq2, vq2 = cached(k[:, perm].contiguous(), v[:, perm].contiguous())
    tc2, _ = run("tc", q, kq2, vq2, 1.0)
    check(tc2, tc, "token permutation")


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("q_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kkw,vkw", [
    (dict(mode="G_SCALE_HEAD_DIM"), dict(mode="G_SCALE_HEAD_DIM")),
    (dict(mode="G_SCALE_HEAD_DIM", symmetric=False), dict(mode="G_TOKEN_HEAD", symmetric=False)),
    (dict(mode="G_TOKEN_HEAD", symmetric=False, group_size=32), dict(mode="G_TOKEN_HEAD", symmetric=False, group_size=32)),
    (dict(mode="G_TOKEN_HEAD", group_size=16, reduce_batch=False), dict(mode="G_HEAD_DIM")),
])
@pytest.mark.parametrize("kb,vb", [(8, 8), (4, 2)])
def test_groupings_whose_k_scale_varies_along_head_dim(D, q_dtype, kkw, vkw, kb, vb):
    """Per-dim and group-wise K: the kernel dequantises K into hi + lo fp16 tiles (two MMAs)."""
    fmt, B, H = "BLHc", 2, 3
    steps = (1, 4, 9, 16, 25, 36, 64, 100, 169)
    kkw, vkw = dict(kkw), dict(vkw)
    km, vm = kkw.pop("mode"), vkw.pop("mode")
    kq, vq = VAR_Q(kb, fmt, km, **kkw), VAR_Q(vb, fmt, vm, **vkw)
    kr, vr = O.OracleVARQ(kb, fmt, km, **kkw), O.OracleVARQ(vb, fmt, vm, **vkw)
    for si, n in enumerate(steps):
        k = O.synthetic_kv((B, n, H, D), fmt, 300 + si, n_outlier=4)
        v = O.synthetic_kv((B, n, H, D), fmt, 400 + si, n_outlier=0)
        kq.append(k.to(DEV)); vq.append(v.to(DEV))
        kd, vd = kr.use_var_q(k), vr.use_var_q(v)
    q = torch.randn((B, 169, H, D), generator=torch.Generator().manual_seed(D + kb)).to(q_dtype)
    scale = 1.0 / D ** 0.5
    out, launches = run("tc", q.to(DEV), kq, vq, scale)
    assert launches == 2          # per-key (or per-step) parameter preparation + the attention kernel
    check(out, O.attention(q, kd, vd, fmt, scale), f"D={D} {q_dtype} K{kkw} V{vkw} {kb}/{vb}")


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("symmetric", [True, False])
def test_all_zero_and_tiny_value_tokens_keep_their_attention_weight(D, symmetric):
    """A token whose V row is all zeros (its scale is the eps clamp) or tiny still takes its share of the
    softmax normaliser: the V scale is folded into P, so such a key must not vanish from the row sum.
    Queries are aligned with those keys so that they carry most of the attention weight."""
    B, H, Lk, Lq = 1, 2, 300, 160
    g = torch.Generator().manual_seed(77 + D)
    k = torch.randn((B, H, Lk, D), generator=g)
    v = torch.randn((B, H, Lk, D), generator=g)
    zero_tok, tiny_tok = [3, 70, 130, 299], [5, 64, 200]
    v[:, :, zero_tok, :] = 0.0
    v[:, :, tiny_tok, :] *= 1e-6
    q = torch.randn((B, H, Lq, D), generator=g)
    q[:, :, :40, :] = 3.0 * k[:, :, 3:4, :] / k[:, :, 3:4, :].norm(dim=-1, keepdim=True) * D ** 0.5      # attends to a zero-V token
    q[:, :, 40:80, :] = 3.0 * k[:, :, 200:201, :] / k[:, :, 200:201, :].norm(dim=-1, keepdim=True) * D ** 0.5   # and to a tiny one
    kq, vq = VAR_Q(8, "BHLc", "G_TOKEN_HEAD", symmetric=symmetric), VAR_Q(8, "BHLc", "G_TOKEN_HEAD", symmetric=symmetric)
    kr, vr = O.OracleVARQ(8, "BHLc", "G_TOKEN_HEAD", symmetric=symmetric), O.OracleVARQ(8, "BHLc", "G_TOKEN_HEAD", symmetric=symmetric)
    kq.append(k.to(DEV)); vq.append(v.to(DEV))
    kd, vd = kr.use_var_q(k), vr.use_var_q(v)
    out, _ = run("tc", q.to(DEV), kq, vq, 1.0 / D ** 0.5)
    check(out, O.attention(q, kd, vd, "BHLc", 1.0 / D ** 0.5).transpose(1, 2), f"zero/tiny V tokens D={D} sym={symmetric}")


@pytest.mark.parametrize("D,kb,vb", [(64, 8, 8), (128, 4, 4)])
def test_per_dim_scales_over_a_long_history_of_steps(D, kb, vb):
    """More appended steps than the step tables of the dequantising mode hold (64): per-dim K scales are then folded
    into the queries step by step, with key tiles cut at the step boundaries (one launch, no preparation)."""
    fmt, B, H = "BLHc", 1, 2
    steps = (1, 2, 3) * 22 + (40, 130)          # 68 steps, 302 tokens
    kq, vq = VAR_Q(kb, fmt, "G_SCALE_HEAD_DIM", symmetric=False), VAR_Q(vb, fmt, "G_SCALE_HEAD_DIM")
    kr, vr = O.OracleVARQ(kb, fmt, "G_SCALE_HEAD_DIM", symmetric=False), O.OracleVARQ(vb, fmt, "G_SCALE_HEAD_DIM")
    for si, n in enumerate(steps):
        k = O.synthetic_kv((B, n, H, D), fmt, 500 + si, n_outlier=4)
        v = O.synthetic_kv((B, n, H, D), fmt, 700 + si, n_outlier=0)
        kq.append(k.to(DEV)); vq.append(v.to(DEV))
        kd, vd = kr.use_var_q(k), vr.use_var_q(v)
    q = torch.randn((B, 150, H, D), generator=torch.Generator().manual_seed(D))
    scale = 1.0 / D ** 0.5
    out, launches = run("tc", q.to(DEV), kq, vq, scale)
    assert launches == 1
    check(out, O.attention(q, kd, vd, fmt, scale), f"68 steps D={D}")


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("kkw,vkw", [
    (dict(mode="G_TOKEN_HEAD", symmetric=False, group_size=32), dict(mode="G_TOKEN_HEAD", symmetric=False, group_size=32)),
    (dict(mode="G_SCALE_HEAD_DIM", symmetric=False), dict(mode="G_SCALE_HEAD_DIM", symmetric=False)),
])
def test_parameters_outside_the_packed_half_converters_bounds(D, kkw, vkw):
    """K values far from zero with a narrow range give zero-points below -512; V scaled up gives scales above 60: the
    preparation kernel flags such tiles and the converters take their fp32 routine (first step only: the second one is
    ordinary data, so flagged and unflagged tiles alternate inside one launch where the parameters are per key)."""
    fmt, B, H = "BLHc", 2, 2
    kkw, vkw = dict(kkw), dict(vkw)
    km, vm = kkw.pop("mode"), vkw.pop("mode")
    kq, vq = VAR_Q(4, fmt, km, **kkw), VAR_Q(4, fmt, vm, **vkw)
    kr, vr = O.OracleVARQ(4, fmt, km, **kkw), O.OracleVARQ(4, fmt, vm, **vkw)
    for si, n in enumerate((200, 150)):
        k = O.synthetic_kv((B, n, H, D), fmt, 900 + si, n_outlier=0)
        v = O.synthetic_kv((B, n, H, D), fmt, 950 + si, n_outlier=0)
        if si == 0:
            k = 5.0 + 0.01 * k            # zero-point = round(-8 - min / scale) is about -1250
            v = 1000.0 * v                # scale = range / 15 is about 500
        kq.append(k.to(DEV)); vq.append(v.to(DEV))
        kd, vd = kr.use_var_q(k), vr.use_var_q(v)
    assert kq._zp_tbl[:, :, :kq._n_rows].abs().max().item() > 512 and vq._scale_tbl[:, :, :vq._n_rows].max().item() > 60
    q = torch.randn((B, 130, H, D), generator=torch.Generator().manual_seed(D))
    scale = 1.0 / D ** 0.5
    out, _ = run("tc", q.to(DEV), kq, vq, scale)
    ref = O.attention(q, kd, vd, fmt, scale)
    out, ref = out.float().cpu(), ref.float().cpu()
    rel = ((out - ref).norm() / ref.norm()).item()
    # the outputs are of the order of V (hundreds): the absolute bound scales with them
    assert rel <= 1e-3 and (out - ref).abs().max().item() <= 2e-3 * max(1.0, ref.abs().max().item()), f"rel-L2 {rel:.3e}"


def test_tensor_core_path_refuses_a_missing_workspace():
    """The preparation streams live in the caller's workspace: without one the call fails with VARQ_ERR_WORKSPACE and
    launches nothing."""
    fmt, B, H, D, lq, lk = "BLHc", 1, 2, 64, 40, 100
    kq, vq = VAR_Q(8, fmt, "G_TOKEN_HEAD"), VAR_Q(8, fmt, "G_TOKEN_HEAD")
    kq.append(torch.randn(B, lk, H, D, device=DEV)); vq.append(torch.randn(B, lk, H, D, device=DEV))
    q = torch.randn(B, lq, H, D, device=DEV)
    out = torch.empty(B, lq, H, D, device=DEV)
    lib = _cabi.lib()
    kc, kp = kq.cache_descriptors()
    vc, vp = vq.cache_descriptors()
    qd = kq._item_desc(q)
    od = _cabi.tensor_desc(out.data_ptr(), _cabi.F32, lq * H * D, H * D, D)
    need = lib.varq_attn_workspace_bytes(B, H, lq, lk, D, 8, 8)
    assert need > 0
    _cabi.force_attn_path("tc")
    n0 = lib.varq_launch_count()
    rc = lib.varq_attn_fwd(qd, kc, vc, kp, vp, B, H, lq, lk, D, 8, 8, 0.125, od, None, 0, _cabi.stream_ptr(q.device))
    assert rc == -4 and b"workspace" in lib.varq_last_error()
    assert lib.varq_launch_count() == n0
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    rc = lib.varq_attn_fwd(qd, kc, vc, kp, vp, B, H, lq, lk, D, 8, 8, 0.125, od, ws.data_ptr(), need, _cabi.stream_ptr(q.device))
    assert rc == 0
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0 and torch.isfinite(out).all()
