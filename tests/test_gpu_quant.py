"""CUDA quantize/pack/dequant against the CPU oracle and the reference-made fixtures.
Bar: bit-exact codes, scales, zero-points and dequantised values for fp32/fp16/bf16 inputs."""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

from oracle import varq_oracle as O
from VAR_Q.pack_unpack import (pack_last_dim_to_int32_triton, unpack_last_dim_from_int32_triton,
                               pack_last_dim_to_int32_python, unpack_last_dim_from_int32_python)
from VAR_Q.quant import VAR_Q

pytestmark = pytest.mark.gpu
DEV = "cuda"


def bits_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    a, b = a.detach().cpu().contiguous(), b.detach().cpu().contiguous()
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    if a.dtype == torch.float32:
        return torch.equal(a.view(torch.int32), b.view(torch.int32))
    return torch.equal(a, b)


# ------------------------------------------------------------------ packing
def test_pack_known_answers(golden_dir):
    kat = json.load(open(os.path.join(golden_dir, "pack_kat.json")))
    for rec in kat["pack"]:
        row = torch.tensor(rec["row"], dtype=torch.int8, device=DEV)
        w, meta = pack_last_dim_to_int32_triton(row, rec["bits"])
        assert [int(x) & 0xFFFFFFFF for x in w.cpu().tolist()] == rec["words"]
        assert meta == rec["meta"]
        assert unpack_last_dim_from_int32_triton(w, meta).cpu().tolist() == rec["row"]


@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("shape", [(3, 5, 7, 64), (2, 9, 20), (1, 1, 1, 5), (4, 33), (0, 16), (100, 17, 128)])
def test_pack_unpack_matches_oracle(bits, shape):
    g = torch.Generator().manual_seed(bits * 1000 + len(shape))
    lo, hi = O.bounds(bits)
    q = torch.randint(lo, hi + 1, shape, generator=g, dtype=torch.int8)
    w_ref, meta_ref = O.pack_words(q, bits)
    w, meta = pack_last_dim_to_int32_python(q.to(DEV), bits)
    assert meta == meta_ref and bits_equal(w, w_ref)
    back = unpack_last_dim_from_int32_python(w, meta)
    assert bits_equal(back, q)


def test_pack_accepts_non_contiguous_and_out_of_range_codes():
    q = torch.arange(-128, 128, dtype=torch.int16).to(torch.int8).repeat(6, 1)      # values wider than 4 bits
    qt = q.t()                                                                       # non-contiguous
    w_ref, _ = O.pack_words(qt.contiguous(), 4)
    w, _ = pack_last_dim_to_int32_triton(qt.to(DEV), 4)
    assert bits_equal(w, w_ref)                                                      # truncated to the field, like the reference


# ------------------------------------------------------------------ fixtures made by the reference
def test_reference_fixtures_bit_exact(golden_dir):
    data = np.load(os.path.join(golden_dir, "quant_small.npz"))
    cases = json.load(open(os.path.join(golden_dir, "quant_small.json")))
    for rec in cases:
        dtype = getattr(torch, rec["dtype"])
        q = VAR_Q(quant_bits=rec["bits"], qkv_format=rec["fmt"], quant_method=rec["mode"])
        n_steps = 1 if rec["mode"] == "G_TENSOR" else len(rec["steps"])   # later G_TENSOR steps: see the defect test
        for si in range(n_steps):
            x = torch.from_numpy(data[f"{rec['key']}_x{si}"]).to(dtype).to(DEV)
            out = q.use_var_q(x)
            tag = f"{rec['key']} {rec['fmt']} {rec['mode']} {rec['bits']}b {rec['dtype']} c={rec['c']} step {si}"
            assert bits_equal(q.cached_item, torch.from_numpy(data[f"{rec['key']}_codes{si}"])), tag
            assert bits_equal(q.cached_scale, torch.from_numpy(data[f"{rec['key']}_scale{si}"])), tag
            assert bits_equal(out, torch.from_numpy(data[f"{rec['key']}_deq{si}"])), tag
            assert out.dtype == torch.float32 and q.cached_item.dtype == torch.int32


def test_behaviour_vectors(golden_dir):
    kat = json.load(open(os.path.join(golden_dir, "pack_kat.json")))
    for rec in kat["quant"]:
        q = VAR_Q(quant_bits=rec["bits"], qkv_format="BLHc", quant_method="G_TOKEN_HEAD")
        q.quant(torch.tensor(rec["x"], dtype=torch.float32, device=DEV).view(1, 1, 1, -1))
        assert int(q.scale.view(-1).view(torch.int32)[0]) == rec["scale_bits"]
        codes = unpack_last_dim_from_int32_triton(q.quantized_item.contiguous(), q._pack_meta)
        assert codes.view(-1).cpu().tolist() == rec["codes"]


def test_c1_shape_hashes(golden_dir):
    rec = json.load(open(os.path.join(golden_dir, "quant_c1.json")))
    x = O.synthetic_kv(tuple(rec["shape"]), rec["fmt"], rec["seed"], n_outlier=4)
    sha = lambda t: hashlib.sha256(t.detach().cpu().contiguous().numpy().tobytes()).hexdigest()
    if sha(x) != rec["x_sha256"]:
        pytest.skip("torch RNG stream differs from the one the fixture was made with")
    q = VAR_Q(quant_bits=rec["bits"], qkv_format=rec["fmt"], quant_method=rec["mode"])
    out = q.use_var_q(x.to(DEV))
    assert sha(q.cached_item) == rec["codes_sha256"]
    assert sha(q.cached_scale) == rec["scale_sha256"]
    assert sha(out) == rec["deq_sha256"]


# ------------------------------------------------------------------ oracle parity, all modes
def run_pair(fmt, mode, bits, steps, B, H, c, dtype=torch.float32, seed=0, strided=False, **ext):
    ref = O.OracleVARQ(bits, fmt, mode, **ext)
    dut = VAR_Q(quant_bits=bits, qkv_format=fmt, quant_method=mode, **ext)
    for si, n in enumerate(steps):
        shape = (B, n, H, c) if fmt == "BLHc" else (B, H, n, c)
        x = O.synthetic_kv(shape, fmt, seed * 97 + si, n_outlier=min(4, c // 4), dtype=dtype)
        xg = x.to(DEV)
        if strided:   # a k/v view cut out of a fused [.., 3, ..] buffer, as the VAR hook passes it
            buf = torch.zeros((*shape[:2], 3, *shape[2:]), dtype=dtype, device=DEV)
            buf[:, :, 1] = xg
            xg = buf.unbind(dim=2)[1]
            assert not xg.is_contiguous()
        want = ref.use_var_q(x)
        got = dut.use_var_q(xg)
        tag = f"{fmt} {mode} {bits}b {ext} step {si} shape {shape} {dtype}"
        assert bits_equal(dut.cached_item, ref.cached_item), "codes " + tag
        assert bits_equal(dut.cached_scale, ref.cached_scale), "scale " + tag
        if not ext.get("symmetric", True):
            assert bits_equal(dut.cached_zero_point, ref.cached_zp), "zero-point " + tag
        assert bits_equal(got, want), "dequant " + tag
        assert bits_equal(dut.dequant_current(), ref.dequant_current()), "dequant_current " + tag
    return dut, ref


@pytest.mark.parametrize("fmt", ["BLHc", "BHLc"])
@pytest.mark.parametrize("mode", O.MODES)
@pytest.mark.parametrize("bits", [2, 4, 8])
def test_modes_multi_step(fmt, mode, bits):
    run_pair(fmt, mode, bits, (1, 4, 9, 16, 25), B=4, H=6, c=64, seed=bits)


@pytest.mark.parametrize("mode", O.MODES)
@pytest.mark.parametrize("symmetric", [True, False])
def test_ragged_head_dim_and_16bit_inputs(mode, symmetric):
    for c, dtype, bits in ((20, torch.float32, 4), (72, torch.bfloat16, 8), (5, torch.float16, 2), (36, torch.float32, 2)):
        run_pair("BLHc", mode, bits, (1, 3, 7), B=3, H=2, c=c, dtype=dtype, seed=c, symmetric=symmetric)


@pytest.mark.parametrize("fmt", ["BLHc", "BHLc"])
@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("group", [None, 32, 16])
@pytest.mark.parametrize("reduce_batch", [True, False])
def test_asymmetric_groupwise(fmt, bits, group, reduce_batch):
    run_pair(fmt, "G_TOKEN_HEAD", bits, (1, 4, 30), B=5, H=3, c=128, seed=7,
             symmetric=False, group_size=group, reduce_batch=reduce_batch)


@pytest.mark.parametrize("mode", ["G_SCALE_HEAD_DIM", "G_TOKEN", "G_SCALE", "G_HEAD_DIM"])
@pytest.mark.parametrize("bits", [4, 8])
def test_asymmetric_other_modes(mode, bits):
    run_pair("BHLc", mode, bits, (2, 5, 17), B=3, H=4, c=64, seed=3, symmetric=False)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("mode", ["G_TOKEN_HEAD", "G_SCALE_HEAD_DIM"])
def test_strided_views_of_a_fused_qkv_buffer(dtype, mode):
    run_pair("BLHc", mode, 8, (1, 4, 9), B=4, H=4, c=64, dtype=dtype, seed=1, strided=True)
    run_pair("BLHc", mode, 4, (1, 4, 9), B=4, H=4, c=64, dtype=dtype, seed=2, strided=True, symmetric=False)


def test_large_batch_takes_the_table_path():
    # 300 samples x 16 threads per row exceed what one CTA holds for a batch-shared group
    run_pair("BLHc", "G_TOKEN_HEAD", 8, (3,), B=300, H=2, c=64, seed=5)
    run_pair("BLHc", "G_TOKEN_HEAD", 4, (3,), B=300, H=2, c=64, seed=6, symmetric=False, group_size=32)


def test_unpacked_int8_storage_and_odd_bit_widths():
    for bits in (3, 5, 8):
        ref = O.OracleVARQ(bits, "BLHc", "G_TOKEN_HEAD")
        dut = VAR_Q(quant_bits=bits, qkv_format="BLHc", quant_method="G_TOKEN_HEAD", pack_to_int32=False)
        x = O.synthetic_kv((2, 6, 3, 32), "BLHc", bits)
        s, z = O.compute_qparams(x, "BLHc", "G_TOKEN_HEAD", bits)
        codes = O.quantize(x, s, z, bits)
        out = dut.use_var_q(x.to(DEV))
        assert dut.cached_item.dtype == torch.int8 and bits_equal(dut.cached_item, codes)
        assert bits_equal(out, O.dequantize(codes, s, z))
    with pytest.raises(AssertionError):
        VAR_Q(quant_bits=3, quant_method="G_TOKEN_HEAD").quant(torch.zeros(1, 1, 1, 8, device=DEV))


def test_g_tensor_replaces_instead_of_duplicating():
    """The reference appends the already re-quantised cache to itself for G_TENSOR
    (1 -> 6 -> 21 tokens for steps of 1, 4, 9).  This build keeps 1 -> 5 -> 14."""
    dut, ref = run_pair("BLHc", "G_TENSOR", 8, (1, 4, 9), B=2, H=3, c=16, seed=9)
    assert dut.cached_item.shape[1] == 14
    defect = O.OracleVARQ(8, "BLHc", "G_TENSOR", g_tensor_append_defect=True)
    for si, n in enumerate((1, 4, 9)):
        defect.use_var_q(O.synthetic_kv((2, n, 3, 16), "BLHc", 9 * 97 + si, n_outlier=4))
    assert defect.cached_item.shape[1] == 21


def test_all_zero_and_constant_groups():
    for symmetric in (True, False):
        x = torch.zeros(2, 3, 2, 64)
        x[:, 1] = 3.25            # a constant token: zero range for the asymmetric case
        run_ref = O.OracleVARQ(4, "BLHc", "G_TOKEN_HEAD", symmetric=symmetric)
        dut = VAR_Q(quant_bits=4, qkv_format="BLHc", quant_method="G_TOKEN_HEAD", symmetric=symmetric)
        want, got = run_ref.use_var_q(x), dut.use_var_q(x.to(DEV))
        assert bits_equal(dut.cached_item, run_ref.cached_item) and bits_equal(dut.cached_scale, run_ref.cached_scale)
        assert bits_equal(got, want)


def test_growth_beyond_capacity_keeps_the_cache():
    ref = O.OracleVARQ(8, "BHLc", "G_SCALE_HEAD_DIM")
    dut = VAR_Q(quant_bits=8, qkv_format="BHLc", quant_method="G_SCALE_HEAD_DIM", max_tokens=8)
    for si in range(70):          # more steps than the initial row table, more tokens than the hint
        x = O.synthetic_kv((2, 2, 3, 32), "BHLc", 1000 + si)
        want, got = ref.use_var_q(x), dut.use_var_q(x.to(DEV))
    assert bits_equal(got, want) and bits_equal(dut.cached_scale, ref.cached_scale)


# ------------------------------------------------------------------ full-size properties
@pytest.mark.parametrize("mode,kw", [("G_TOKEN_HEAD", {}), ("G_SCALE_HEAD_DIM", {}),
                                     ("G_TOKEN_HEAD", dict(symmetric=False, group_size=32, reduce_batch=False))])
def test_full_size_step_properties(mode, kw):
    """VAR-d30 last step (B2=128, l=1024, H=30, c=64, fp32 = 1 GB): too big for the CPU oracle to
    finish in seconds, so check properties: codes in range, |x - deq| <= scale/2 inside the group
    range, and re-quantising the dequantised tensor with the same parameters is the identity."""
    B, n, H, c, bits = 128, 1024, 30, 64, 4
    g = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn((B, n, H, c), generator=g, device=DEV)
    x[..., :4] *= 20
    q = VAR_Q(quant_bits=bits, qkv_format="BLHc", quant_method=mode, **kw)
    deq = q.use_var_q(x)
    codes = unpack_last_dim_from_int32_triton(q.cached_item.contiguous(), q._pack_meta)
    assert int(codes.min()) >= -8 and int(codes.max()) <= 7
    s = q.cached_scale
    s = s if s.shape[-1] in (1, c) else s.repeat_interleave(c // s.shape[-1], dim=-1)
    err = (deq - x).abs()
    assert bool((err <= s * 0.5 * 1.0001 + 1e-30).all())
    # idempotence on a slice the oracle can handle: same codes when fed the dequantised values
    sub = deq[:2, :64].cpu()
    if mode == "G_TOKEN_HEAD" and kw.get("reduce_batch", True) is False:
        r = O.OracleVARQ(bits, "BLHc", mode, **kw)
        r.use_var_q(x[:2, :64].cpu())
        assert bits_equal(q.cached_item[:2, :64], r.cached_item)


@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("symmetric", [True, False])
def test_rounding_ties_and_their_neighbours(bits, symmetric):
    """Quotients at and within a few ulps of k + 1/2, for many scales: the kernel multiplies by a
    reciprocal and must still reproduce round-half-even of the fp32-rounded true quotient."""
    g = torch.Generator().manual_seed(bits)
    lo, hi = O.bounds(bits)
    rows, c = 4096, 64
    amax = torch.rand(rows, generator=g) * 10 ** (torch.rand(rows, generator=g) * 8 - 4)      # 1e-4 .. 1e4
    span = float(hi) if symmetric else float((1 << bits) - 1)
    s = amax / span
    k = torch.randint(lo, hi, (rows, c), generator=g).float() + 0.5
    x = (k * s[:, None]).clamp(-amax[:, None], amax[:, None])
    ulps = torch.randint(-3, 4, (rows, c), generator=g, dtype=torch.int32)
    x = (x.view(torch.int32) + ulps).view(torch.float32)
    x = torch.where(x.abs() > amax[:, None], torch.sign(x) * amax[:, None], x)
    x[:, 0] = amax                      # pins max |x| (and max) of the row
    x[:, 1] = -amax if symmetric else 0.0 * amax
    x = x.view(1, rows, 1, c)
    ref = O.OracleVARQ(bits, "BLHc", "G_TOKEN_HEAD", symmetric=symmetric)
    dut = VAR_Q(quant_bits=bits, qkv_format="BLHc", quant_method="G_TOKEN_HEAD", symmetric=symmetric)
    want, got = ref.use_var_q(x), dut.use_var_q(x.to(DEV))
    assert bits_equal(dut.cached_scale, ref.cached_scale)
    assert bits_equal(dut.cached_item, ref.cached_item)
    assert bits_equal(got, want)
    # the same rows through the two-kernel path (per-tensor statistics)
    ref2, dut2 = O.OracleVARQ(bits, "BLHc", "G_SCALE", symmetric=symmetric), VAR_Q(bits, "BLHc", "G_SCALE", symmetric=symmetric)
    assert bits_equal(dut2.use_var_q(x.to(DEV)), ref2.use_var_q(x))
    assert bits_equal(dut2.cached_item, ref2.cached_item)


@pytest.mark.parametrize("B", [8, 16, 64])
@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("symmetric,group", [(True, None), (False, None), (False, 32), (True, 16)])
def test_batch_shared_groups_register_resident_path(B, bits, symmetric, group):
    """Batch sizes that fill every register slot of the single-pass kernel (B = lanes x vectors)."""
    for fmt, dtype in (("BLHc", torch.float32), ("BHLc", torch.bfloat16)):
        run_pair(fmt, "G_TOKEN_HEAD", bits, (1, 5, 12), B=B, H=4, c=64, dtype=dtype, seed=B + bits,
                 symmetric=symmetric, group_size=group)
    run_pair("BLHc", "G_TOKEN_HEAD", bits, (3, 4), B=B, H=2, c=128, dtype=torch.float16, seed=B, strided=True,
             symmetric=symmetric, group_size=group)


# ------------------------------------------------------------------ compact cache save / load, statistics
@pytest.mark.parametrize("mode,kw", [("G_TOKEN_HEAD", dict(symmetric=False, group_size=32)), ("G_SCALE_HEAD_DIM", {}), ("G_HEAD_DIM", {})])
def test_cache_round_trips_through_save_and_load(mode, kw, tmp_path):
    dut, ref = run_pair("BLHc", mode, 4, (1, 4, 9), B=3, H=2, c=64, seed=11, **kw)
    path = str(tmp_path / "cache.pt")
    dut.save(path)
    other = VAR_Q(quant_bits=4, qkv_format="BLHc", quant_method=mode, **kw).load(path)
    assert other.n_tokens == 14 and bits_equal(other.cached_item, ref.cached_item) and bits_equal(other.cached_scale, ref.cached_scale)
    assert bits_equal(other.dequant_all(), ref.dequant_all())
    x = O.synthetic_kv((3, 16, 2, 64), "BLHc", 99)
    assert bits_equal(other.use_var_q(x.to(DEV)), ref.use_var_q(x))           # appending to a restored cache continues it
    with pytest.raises(ValueError):
        VAR_Q(quant_bits=8, qkv_format="BLHc", quant_method=mode, **kw).load(path)


def test_debug_statistics_rows_and_csv(tmp_path):
    q = VAR_Q(quant_bits=4, qkv_format="BLHc", quant_method="G_TOKEN_HEAD", blk_idx=5, debug=True)
    for si, n in enumerate((2, 7)):
        x = O.synthetic_kv((2, n, 3, 64), "BLHc", 40 + si).to(DEV)
        q.use_var_q(x)
    rows = q.debug_rows
    assert len(rows) == 2 and rows[1]["cached_tokens"] == 9 and rows[0]["blk_idx"] == 5
    assert 0.0 < rows[0]["rel_l2_error"] < 0.5 and rows[0]["max_abs_error"] <= rows[0]["scale_max"] * 0.5 * 1.0001
    path = str(tmp_path / "stats.csv")
    q.write_statistics_csv(path)
    lines = open(path).read().strip().splitlines()
    assert len(lines) == 3 and lines[0].startswith("blk_idx,step_tokens,cached_tokens")
