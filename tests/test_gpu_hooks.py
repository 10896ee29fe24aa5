"""The hook-level replacement (LayerKV) inside a stand-in attention layer shaped like the VAR and
Infinity SelfAttention: fused QKV projection, L2-normalised q/k, per-scale steps."""
import os

import pytest
import torch

from oracle import varq_oracle as O
from VAR_Q.config_loader import load_varq_config
from VAR_Q.hooks import LayerKV

pytestmark = pytest.mark.gpu
DEV = "cuda"
CFG_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "var-q_b200", "VAR_Q")


class StandInAttention(torch.nn.Module):
    """qkv = x W^T viewed [B, L, 3, H, c]; flash layout ('BLHc') or SDPA layout ('BHLc')."""

    def __init__(self, width, heads, fmt, q_bits, method, l2=True):
        super().__init__()
        self.heads, self.c, self.fmt, self.l2 = heads, width // heads, fmt, l2
        self.mat_qkv = torch.nn.Linear(width, 3 * width, bias=False)
        self.q_bits, self.quant_method, self.qkv_format, self.enable_quantization, self.block_idx = q_bits, method, fmt, True, 3
        self.scale = 1.0 if l2 else 0.25 / self.c ** 0.5

    def qkv(self, x):
        B, L, _ = x.shape
        qkv = self.mat_qkv(x).view(B, L, 3, self.heads, self.c)
        q, k, v = qkv.unbind(dim=2) if self.fmt == "BLHc" else qkv.permute(2, 0, 3, 1, 4).unbind(dim=0)
        if self.l2:
            q = torch.nn.functional.normalize(q.float(), dim=-1) * 4.0
            k = torch.nn.functional.normalize(k.float(), dim=-1)
        return q, k, v


@pytest.mark.parametrize("fmt", ["BLHc", "BHLc"])
@pytest.mark.parametrize("method,bits", [("G_SCALE_HEAD_DIM", 8), ("G_TOKEN_HEAD", 4)])
@pytest.mark.parametrize("l2", [True, False])
def test_fused_step_matches_oracle_and_reference_route(fmt, method, bits, l2):
    torch.manual_seed(0)
    layer = StandInAttention(256, 4, fmt, bits, method, l2).to(DEV).to(torch.bfloat16)
    fused, route = LayerKV.from_module(layer), LayerKV.from_module(layer)
    kr, vr = O.OracleVARQ(bits, fmt, method), O.OracleVARQ(bits, fmt, method)
    assert fused.k_quant.cur_blk_idx == 3
    for n in (1, 4, 9, 16, 25, 36):
        x = torch.randn(2, n, 256, device=DEV, dtype=torch.bfloat16)
        q, k, v = layer.qkv(x)                           # k, v may be strided views of the qkv buffer
        out = fused.step(q, k, v, layer.scale, out_dtype=torch.bfloat16)
        alt = route.step_reference_route(q, k, v, layer.scale, torch.bfloat16)
        ref = O.attention(q.float().cpu(), kr.use_var_q(k.float().cpu()), vr.use_var_q(v.float().cpu()), fmt, layer.scale)
        ref = ref if fmt == "BLHc" else ref.transpose(1, 2)
        assert out.shape == (2, n, 4, 64) and out.dtype == torch.bfloat16
        # bf16 output rounding (2^-9 relative) on top of the kernel tolerance
        assert (out.float().cpu() - ref).abs().max() <= 2e-3 + 4e-3 * ref.abs().max()
        assert (alt.float().cpu() - ref).abs().max() <= 2e-2 * max(1.0, ref.abs().max().item())
    assert fused.n_tokens == 91


def test_from_config_resolves_per_tensor_settings():
    cfg = load_varq_config(os.path.join(CFG_DIR, "VAR-d30-int4-asym.json"))
    kv = LayerKV.from_config(cfg, max_tokens=64)
    assert kv.k_quant.quant_method == "G_SCALE_HEAD_DIM" and not kv.k_quant.symmetric
    assert kv.v_quant.quant_method == "G_TOKEN_HEAD" and kv.v_quant.group_size == 64
    q = torch.randn(2, 5, 3, 64, device=DEV)
    out = kv.step(q, torch.randn(2, 5, 3, 64, device=DEV), torch.randn(2, 5, 3, 64, device=DEV), 0.125)
    assert out.shape == (2, 5, 3, 64) and torch.isfinite(out).all()
    raw = load_varq_config(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_configs", "VAR-raw.json"))
    assert LayerKV.from_config(raw) is None
    kv.set_format("BHLc")
    assert kv.k_quant.dim_cat == 2
