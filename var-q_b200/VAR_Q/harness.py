"""A stand-in for the model loop around the hook, for whole-loop throughput numbers.

The reference measures generation through ``VAR.autoregressive_infer_cfg`` (VAR/models/var.py:130-193): CFG doubles the
batch, ``kv_caching(True)`` is switched on in every block, and for each scale of the schedule the new token map runs
through all blocks, each of which projects QKV, takes the hook (quantize + cache + attention) and applies its MLP.
The reference's model classes, tokenizer and checkpoints do not travel with this package, so ``StandInVAR`` rebuilds
only that skeleton with randomly initialised torch layers of the same shapes: LayerNorm -> attention (with
``VAR_Q.hooks.install``) -> LayerNorm -> 4x MLP per block, a random token map per scale in place of sampling and
embedding.  It exists to time the hot path where it runs in practice -- between GEMMs, launched from Python or
replayed as one CUDA graph -- not to generate images.
"""
import math
from typing import Optional, Sequence

import torch

from .hooks import install


class StandInSelfAttention(torch.nn.Module):
    """Carries the attributes ``hooks.install`` reads (the reference class's, VAR/models/basic_var.py:73-117)."""

    def __init__(self, width: int, heads: int, block_idx: int, q_bits: int, quant_method: str, attn_l2_norm: bool = True):
        super().__init__()
        self.block_idx, self.num_heads, self.head_dim = block_idx, heads, width // heads
        self.attn_l2_norm, self.q_bits, self.quant_method, self.qkv_format = attn_l2_norm, q_bits, quant_method, 'BLHc'
        self.enable_quantization = True
        if attn_l2_norm:
            self.scale = 1
            self.scale_mul_1H11 = torch.nn.Parameter(torch.full((1, heads, 1, 1), 4.0).log())
            self.max_scale_mul = math.log(100)
        else:
            self.scale = 0.25 / math.sqrt(self.head_dim)
        self.mat_qkv = torch.nn.Linear(width, 3 * width, bias=False)
        self.q_bias, self.v_bias = torch.nn.Parameter(torch.zeros(width)), torch.nn.Parameter(torch.zeros(width))
        self.register_buffer('zero_k_bias', torch.zeros(width))
        self.proj, self.proj_drop = torch.nn.Linear(width, width), torch.nn.Identity()
        self.caching, self.k_quant, self.v_quant = False, None, None

    def kv_caching(self, enable: bool):
        self.caching = enable
        self.k_quant = self.v_quant = None

    def forward(self, x, attn_bias=None):
        raise RuntimeError("StandInSelfAttention only runs with kv_caching(True) and the installed packed-cache route")


class StandInBlock(torch.nn.Module):
    def __init__(self, width, heads, block_idx, q_bits, quant_method, max_tokens, k_kwargs, v_kwargs):
        super().__init__()
        self.ln1, self.ln2 = torch.nn.LayerNorm(width), torch.nn.LayerNorm(width)
        self.attn = install(StandInSelfAttention(width, heads, block_idx, q_bits, quant_method), max_tokens, k_kwargs, v_kwargs)
        self.fc1, self.fc2 = torch.nn.Linear(width, 4 * width), torch.nn.Linear(4 * width, width)

    def forward(self, x):
        x = x + self.attn(self.ln1(x), None)
        return x + self.fc2(torch.nn.functional.gelu(self.fc1(self.ln2(x)), approximate='tanh'))


class StandInVAR(torch.nn.Module):
    def __init__(self, depth: int = 16, width: int = 1024, heads: int = 16,
                 patch_nums: Sequence[int] = (1, 2, 3, 4, 5, 6, 8, 10, 13, 16), q_bits: int = 8,
                 quant_method: str = 'G_TOKEN_HEAD', k_kwargs: Optional[dict] = None, v_kwargs: Optional[dict] = None):
        super().__init__()
        self.width, self.patch_nums = width, tuple(patch_nums)
        total = sum(p * p for p in patch_nums)
        self.blocks = torch.nn.ModuleList(StandInBlock(width, heads, i, q_bits, quant_method, total, k_kwargs, v_kwargs)
                                          for i in range(depth))

    @torch.inference_mode()
    def generate(self, token_maps: Sequence[torch.Tensor]) -> torch.Tensor:
        """One pass over the scale schedule.  ``token_maps[i]`` is the (CFG-doubled) input of scale i, [2B, pn_i^2, width];
        returns the last scale's hidden state."""
        for b in self.blocks:
            b.attn.kv_caching(True)
        x = None
        for tm in token_maps:
            x = tm
            for b in self.blocks:
                x = b(x)
        for b in self.blocks:
            b.attn.kv_caching(False)
        return x

    def token_maps(self, batch: int, device, dtype=torch.bfloat16, seed: int = 0):
        g = torch.Generator(device=device).manual_seed(seed)
        return [torch.randn((2 * batch, p * p, self.width), generator=g, device=device, dtype=torch.float32).to(dtype)
                for p in self.patch_nums]
