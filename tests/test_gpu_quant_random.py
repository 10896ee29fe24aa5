"""Seeded random shapes, groupings, bit widths, layouts, dtypes and multi-step appends:
`use_var_q` (quantize + pack + cache + unpack + dequantize on the GPU) must equal the CPU oracle
bit for bit, whichever of the quantize kernels (row kernels, two-pass tables) and dequant kernels
the shape selects."""
import random

import pytest
import torch

from oracle import varq_oracle as O
from VAR_Q.quant import VAR_Q

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_use_var_q_matches_the_oracle_on_random_cases(seed):
    rng = random.Random(seed)
    for it in range(40):
        fmt = rng.choice(["BLHc", "BHLc"])
        mode = rng.choice(["G_TENSOR", "G_SCALE_HEAD_DIM", "G_HEAD_DIM", "G_SCALE", "G_TOKEN", "G_TOKEN_HEAD"])
        bits = rng.choice([2, 4, 8])
        B, H, D = rng.choice([1, 2, 3, 8, 17, 64]), rng.choice([1, 2, 5, 16, 30]), rng.choice([16, 32, 64, 128, 48])
        kw = {}
        if rng.random() < 0.4:
            kw["symmetric"] = False
        if mode in ("G_TOKEN", "G_TOKEN_HEAD") and rng.random() < 0.3:
            kw["reduce_batch"] = False
        if mode == "G_TOKEN_HEAD" and rng.random() < 0.3 and D % 16 == 0:
            kw["group_size"] = 16
        dtype = rng.choice([torch.float32, torch.bfloat16, torch.float16])
        steps = [rng.choice([1, 3, 16, 61, 200]) for _ in range(rng.choice([1, 2, 3]))]
        if mode == "G_TENSOR":
            steps = steps[:1]
        ours, ref = VAR_Q(bits, fmt, mode, **kw), O.OracleVARQ(bits, fmt, mode, **kw)
        g = torch.Generator().manual_seed(seed * 1000 + it)
        tag = f"it={it} {fmt} {mode} {bits}b B{B} H{H} D{D} {kw} {dtype} steps={steps}"
        for n in steps:
            shape = (B, n, H, D) if fmt == "BLHc" else (B, H, n, D)
            x = (torch.randn(shape, generator=g) * rng.choice([0.05, 1.0, 30.0]) + rng.choice([0.0, 0.0, 2.5])).to(dtype)
            a = ours.use_var_q(x.to(DEV)).float().cpu()
            b = ref.use_var_q(x).float()
            assert a.shape == b.shape, tag
            assert torch.equal(a, b), f"{tag} at step of {n} tokens: max diff {(a - b).abs().max().item():.3e}"
