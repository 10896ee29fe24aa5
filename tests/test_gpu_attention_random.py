"""Seeded random shapes, groupings, bit widths, layouts and query dtypes: the tensor-core kernel
(more than 16 queries) and the streaming kernel (1-16 queries) against the general CUDA-core kernel.
Both sides read the same packed cache, so the comparison isolates the attention arithmetic.
Tolerance: max-abs 2e-3 (relative to max(1, max|ref|)) and relative L2 1e-3; outputs whose
magnitude is below 1e-2 are held to the absolute bound only (fp16 operand rounding is relative to
the V values, not to a near-cancelling output)."""
import random

import pytest
import torch

from VAR_Q import _cabi
from VAR_Q.attention import attend_cached
from VAR_Q.quant import VAR_Q

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _auto_path_afterwards():
    yield
    _cabi.force_attn_path(None)


def _case(rng, it, lq_choices):
    D = rng.choice([64, 128])
    fmt = rng.choice(["BLHc", "BHLc"])
    B, H = rng.choice([1, 2, 3]), rng.choice([1, 2, 5])
    kb, vb = rng.choice([2, 4, 8]), rng.choice([2, 4, 8])
    mode = rng.choice(["G_TOKEN_HEAD", "G_TOKEN_HEAD", "G_SCALE_HEAD_DIM", "G_HEAD_DIM", "G_TOKEN", "G_SCALE", "G_TENSOR"])
    kw = {}
    if rng.random() < 0.4:
        kw["symmetric"] = False
    if mode == "G_TOKEN_HEAD" and rng.random() < 0.3:
        kw["group_size"] = rng.choice([16, 32])
    steps = [rng.choice([1, 7, 33, 64, 100, 129, 200, 333]) for _ in range(rng.choice([1, 2, 4]))]
    if mode == "G_TENSOR":
        steps = steps[:1]
    lq = rng.choice(lq_choices)
    gain = rng.choice([0.125, 0.125, 1.0, 4.0])      # large gains exercise the reference-maximum updates
    q_dtype = rng.choice([torch.float32, torch.bfloat16, torch.float16])
    g = torch.Generator().manual_seed(it)
    kq, vq = VAR_Q(kb, fmt, mode, **kw), VAR_Q(vb, fmt, mode, **kw)
    for n in steps:
        shape = (B, n, H, D) if fmt == "BLHc" else (B, H, n, D)
        k = torch.randn(shape, generator=g) * rng.choice([0.1, 1.0, 5.0])
        v = torch.randn(shape, generator=g) * rng.choice([0.01, 1.0, 3.0])
        if rng.random() < 0.3:
            v = v + 2.0
        if rng.random() < 0.3:
            k[..., :3] *= 8.0
        kq.append(k.to(DEV)); vq.append(v.to(DEV))
    q_shape = (B, lq, H, D) if fmt == "BLHc" else (B, H, lq, D)
    q = torch.randn(q_shape, generator=g).to(q_dtype).to(DEV)
    tag = f"it={it} D={D} {fmt} B{B} H{H} k{kb} v{vb} {mode} {kw} steps={steps} Lq={lq} gain={gain} {q_dtype}"
    return q, kq, vq, gain / D ** 0.5 * 8, tag


def _compare(path, q, kq, vq, scale, tag):
    outs = {}
    for p in (path, "small"):
        _cabi.force_attn_path(p)
        outs[p] = attend_cached(q, kq, vq, scale, out_dtype=torch.float32).float()
    torch.cuda.synchronize()
    status = _cabi.device_status()
    assert status == 0, f"{tag}: a kernel wait expired (code {status})"
    a, b = outs[path], outs["small"]
    assert torch.isfinite(a).all(), tag
    err = (a - b).abs().max().item()
    rel = ((a - b).norm() / b.norm().clamp_min(1e-30)).item()
    ref_max = b.abs().max().item()
    assert err <= 2e-3 * max(1.0, ref_max), f"{tag}: max-abs {err:.3e} (max|ref| {ref_max:.3f})"
    assert rel <= 1e-3 or ref_max < 1e-2, f"{tag}: rel-L2 {rel:.3e}"


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_tensor_core_kernel_on_random_cases(seed):
    rng = random.Random(seed)
    for it in range(40):
        _compare("tc", *_case(rng, seed * 1000 + it, [9, 16, 64, 127, 128, 129, 256, 300]))


@pytest.mark.parametrize("seed", [3, 4])
def test_streaming_kernel_on_random_cases(seed):
    rng = random.Random(seed)
    for it in range(40):
        _compare("stream", *_case(rng, seed * 1000 + it, [1, 2, 4, 5, 8, 9, 13, 16]))
