"""The fused producer kernel (L2-normalise q / k + column statistics in one read), the quantize call that starts from its
statistics, and `hooks.install` on a module shaped like the reference's VAR SelfAttention.

Bars: normalised q / k within fp32 rounding of torch.nn.functional.normalize; packed codes, scales and zero-points
bit-exact against the oracle run on the values the kernel itself emitted; installed forward within the attention
tolerance (plus the output dtype's rounding) of the reference's sequence restated with the oracle."""
import math

import pytest
import torch

from oracle import varq_oracle as O
from VAR_Q import _cabi
from VAR_Q.hooks import LayerKV, install, normalise_qk
from VAR_Q.quant import VAR_Q

pytestmark = pytest.mark.gpu
DEV = "cuda"


def bits_equal(a, b):
    a, b = a.detach().cpu().contiguous(), b.detach().cpu().contiguous()
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    return torch.equal(a.view(torch.int32), b.view(torch.int32)) if a.dtype == torch.float32 else torch.equal(a, b)


def _views(fmt, B, L, H, c, dtype, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    qkv = torch.randn((B, L, 3, H, c), generator=g, device=DEV)
    qkv[..., :3] *= 5.0
    qkv = qkv.to(dtype)
    return qkv.unbind(dim=2) if fmt == "BLHc" else qkv.permute(2, 0, 3, 1, 4).unbind(dim=0)


@pytest.mark.parametrize("fmt", ["BLHc", "BHLc"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("c", [64, 128, 40])
def test_normalised_q_and_k_match_torch(fmt, dtype, c):
    B, L, H = 3, 37, 5
    q, k, v = _views(fmt, B, L, H, c, dtype, seed=c)
    kq, vq = VAR_Q(8, fmt, "G_TOKEN_HEAD"), VAR_Q(8, fmt, "G_TOKEN_HEAD")         # no statistics wanted
    mul = torch.linspace(1.0, 7.0, H, device=DEV)
    qn, kn, ks, vs = normalise_qk(q, k, v, kq, vq, scale_mul=mul)
    assert ks is None and vs is None and qn.dtype == torch.float32 and qn.shape == q.shape
    shape = (1, 1, H, 1) if fmt == "BLHc" else (1, H, 1, 1)
    q_ref = torch.nn.functional.normalize(q.float(), dim=-1) * mul.view(shape)
    k_ref = torch.nn.functional.normalize(k.float(), dim=-1)
    assert torch.allclose(qn, q_ref, rtol=4e-7, atol=1e-30) and torch.allclose(kn, k_ref, rtol=4e-7, atol=1e-30)
    zero = torch.zeros_like(q)                                                       # zero rows: 0 / eps = 0, no NaN
    qz, kz, _, _ = normalise_qk(zero, zero, v, kq, vq)
    assert float(qz.abs().max()) == 0.0 and float(kz.abs().max()) == 0.0


@pytest.mark.parametrize("fmt", ["BLHc", "BHLc"])
@pytest.mark.parametrize("k_cfg,v_cfg", [
    ((4, "G_SCALE_HEAD_DIM", dict(symmetric=False)), (8, "G_SCALE_HEAD_DIM", {})),
    ((8, "G_SCALE_HEAD_DIM", {}), (4, "G_TOKEN_HEAD", dict(symmetric=False))),       # V has no use for statistics
    ((2, "G_SCALE", {}), (4, "G_SCALE", dict(symmetric=False))),
])
def test_quantize_from_the_fused_statistics_is_bit_exact(fmt, k_cfg, v_cfg):
    B, H, c = 4, 6, 64
    (kb, km, kkw), (vb, vm, vkw) = k_cfg, v_cfg
    kq, vq = VAR_Q(kb, fmt, km, **kkw), VAR_Q(vb, fmt, vm, **vkw)
    kr, vr = O.OracleVARQ(kb, fmt, km, **kkw), O.OracleVARQ(vb, fmt, vm, **vkw)
    lib = _cabi.lib()
    for si, L in enumerate((1, 9, 100)):
        q, k, v = _views(fmt, B, L, H, c, torch.bfloat16, seed=10 + si)
        qn, kn, ks, vs = normalise_qk(q, k, v, kq, vq)
        assert ks is not None and (vs is not None) == (vm != "G_TOKEN_HEAD")
        n0 = lib.varq_launch_count()
        kq.append(kn, ks)
        assert lib.varq_launch_count() - n0 == 2           # finalize + apply: no statistics kernel
        vq.append(v, vs)
        kr.use_var_q(kn.cpu()); vr.use_var_q(v.cpu())       # the oracle sees the values the kernel emitted
        for dut, ref, name in ((kq, kr, "K"), (vq, vr, "V")):
            assert bits_equal(dut.cached_item, ref.cached_item), f"{name} codes step {si}"
            assert bits_equal(dut.cached_scale, ref.cached_scale), f"{name} scales step {si}"
            if ref.cached_zp is not None:
                assert bits_equal(dut.cached_zero_point, ref.cached_zp), f"{name} zero-points step {si}"


class VarShapedAttention(torch.nn.Module):
    """The attributes and the forward of the reference's VAR SelfAttention (VAR/models/basic_var.py:73-164), minus
    drop-out and the optional attention libraries: what `install` expects to find."""

    def __init__(self, width, heads, q_bits, method, l2=True, block_idx=2):
        super().__init__()
        self.block_idx, self.num_heads, self.head_dim = block_idx, heads, width // heads
        self.attn_l2_norm, self.q_bits, self.quant_method, self.qkv_format, self.enable_quantization = l2, q_bits, method, "BHLc", True
        if l2:
            self.scale = 1
            self.scale_mul_1H11 = torch.nn.Parameter(torch.full((1, heads, 1, 1), 4.0).log())
            self.max_scale_mul = math.log(100)
        else:
            self.scale = 0.25 / math.sqrt(self.head_dim)
        self.mat_qkv = torch.nn.Linear(width, width * 3, bias=False)
        self.q_bias, self.v_bias = torch.nn.Parameter(torch.randn(width) * 0.1), torch.nn.Parameter(torch.randn(width) * 0.1)
        self.register_buffer("zero_k_bias", torch.zeros(width))
        self.proj, self.proj_drop = torch.nn.Linear(width, width), torch.nn.Identity()
        self.caching, self.k_quant, self.v_quant = False, None, None

    def kv_caching(self, enable):
        self.caching = enable
        self.k_quant = self.v_quant = None

    def forward(self, x, attn_bias=None):
        raise AssertionError("the installed forward must take over while caching with quantization is on")


def _reference_forward(m, x, kr, vr):
    """The reference's sequence: the module's own QKV projection (on the GPU, so that both sides quantize identical
    activations), then on the CPU fp32 L2-normalisation, oracle quantizers and fp32 attention, then the module's proj."""
    B, L, C = x.shape
    qkv = torch.nn.functional.linear(x, m.mat_qkv.weight, torch.cat((m.q_bias, m.zero_k_bias, m.v_bias))).view(B, L, 3, m.num_heads, m.head_dim)
    main_type = qkv.dtype
    q, k, v = qkv.cpu().unbind(dim=2)
    if m.attn_l2_norm:
        mul = m.scale_mul_1H11.detach().cpu().clamp_max(m.max_scale_mul).exp().transpose(1, 2)
        q, k = torch.nn.functional.normalize(q.float(), dim=-1) * mul, torch.nn.functional.normalize(k.float(), dim=-1)
    o = O.attention(q, kr.use_var_q(k), vr.use_var_q(v), "BLHc", float(m.scale))
    return m.proj(o.reshape(B, L, C).to(DEV).to(main_type))


@pytest.mark.parametrize("method,bits", [("G_SCALE_HEAD_DIM", 8), ("G_TOKEN_HEAD", 4)])
@pytest.mark.parametrize("l2", [True, False])
def test_install_takes_over_a_var_shaped_module_under_autocast(method, bits, l2):
    torch.manual_seed(1)
    width, heads = 256, 4
    m = install(VarShapedAttention(width, heads, bits, method, l2).to(DEV), max_tokens=128)
    kr, vr = O.OracleVARQ(bits, "BLHc", method), O.OracleVARQ(bits, "BLHc", method)
    m.kv_caching(True)
    assert isinstance(m._varq_kv, LayerKV) and m._varq_kv.k_quant.cur_blk_idx == 2
    with torch.inference_mode(), torch.autocast("cuda", dtype=torch.bfloat16):
        for n in (1, 4, 9, 16, 25, 36):
            x = torch.randn(2, n, width, device=DEV)
            out = m(x, None)
            ref = _reference_forward(m, x, kr, vr).float()
            assert out.shape == (2, n, width)
            assert (out.float() - ref).abs().max() <= 0.03 * max(1.0, ref.abs().max().item()), f"step of {n} tokens"
    assert m._varq_kv.n_tokens == 91
    m.kv_caching(False)
    assert m._varq_kv is None
    with pytest.raises(AssertionError):
        m(torch.randn(1, 2, width, device=DEV), None)            # not caching: the original forward is called


def test_stand_in_block_loop_runs_eagerly_and_as_a_cuda_graph():
    from VAR_Q.harness import StandInVAR
    torch.manual_seed(3)
    model = StandInVAR(depth=2, width=128, heads=2, patch_nums=(1, 2, 3, 5), q_bits=4, quant_method="G_SCALE_HEAD_DIM",
                       k_kwargs=dict(symmetric=False)).to(DEV).to(torch.bfloat16)
    maps = model.token_maps(3, DEV)
    eager = model.generate(maps).clone()
    assert eager.shape == (6, 25, 128) and torch.isfinite(eager.float()).all()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        model.generate(maps)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = model.generate(maps)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    assert _cabi.device_status() == 0
