"""The CPU oracle against outputs of the reference itself (fixtures in tests/golden)."""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

from oracle import varq_oracle as O


def _load(golden_dir, name):
    with open(os.path.join(golden_dir, name)) as f:
        return json.load(f)


def test_pack_known_answers(golden_dir):
    kat = _load(golden_dir, "pack_kat.json")
    for rec in kat["pack"]:
        w, meta = O.pack_words(torch.tensor(rec["row"], dtype=torch.int8), rec["bits"])
        assert [int(x) & 0xFFFFFFFF for x in w.tolist()] == rec["words"]
        assert meta == rec["meta"]
        assert O.unpack_words(w, meta).tolist() == rec["row"]


def test_quantizer_behaviour_vectors(golden_dir):
    kat = _load(golden_dir, "pack_kat.json")
    for rec in kat["quant"]:
        x = torch.tensor(rec["x"], dtype=torch.float32).view(1, 1, 1, -1)
        s, z = O.compute_qparams(x, "BLHc", "G_TOKEN_HEAD", rec["bits"])
        assert int(s.view(-1).view(torch.int32)[0]) == rec["scale_bits"]
        assert O.quantize(x, s, z, rec["bits"]).view(-1).tolist() == rec["codes"]


def _cases(golden_dir):
    return _load(golden_dir, "quant_small.json")


def test_small_sequences_bit_exact(golden_dir):
    data = np.load(os.path.join(golden_dir, "quant_small.npz"))
    cases = _cases(golden_dir)
    assert len(cases) >= 36
    for rec in cases:
        dtype = getattr(torch, rec["dtype"])
        q = O.OracleVARQ(rec["bits"], rec["fmt"], rec["mode"], g_tensor_append_defect=True)
        for si in range(len(rec["steps"])):
            x = torch.from_numpy(data[f"{rec['key']}_x{si}"]).to(dtype)
            out = q.use_var_q(x)
            tag = f"{rec['key']} {rec['fmt']} {rec['mode']} {rec['bits']}b step {si}"
            assert np.array_equal(q.cached_item.numpy(), data[f"{rec['key']}_codes{si}"]), tag
            ref_scale = data[f"{rec['key']}_scale{si}"]
            assert q.cached_scale.shape == ref_scale.shape, tag
            assert np.array_equal(q.cached_scale.contiguous().numpy().view(np.int32), ref_scale.view(np.int32)), tag
            assert np.array_equal(out.numpy().view(np.int32), data[f"{rec['key']}_deq{si}"].view(np.int32)), tag


def test_c1_shape_hashes(golden_dir):
    rec = _load(golden_dir, "quant_c1.json")
    x = O.synthetic_kv(tuple(rec["shape"]), rec["fmt"], rec["seed"], n_outlier=4)
    sha = lambda t: hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()
    if sha(x) != rec["x_sha256"]:
        pytest.skip("torch RNG stream differs from the one the fixture was made with")
    q = O.OracleVARQ(rec["bits"], rec["fmt"], rec["mode"])
    out = q.use_var_q(x)
    assert sha(q.cached_item) == rec["codes_sha256"]
    assert sha(q.cached_scale) == rec["scale_sha256"]
    assert sha(out) == rec["deq_sha256"]


def test_extension_reduces_to_reference_modes():
    x = O.synthetic_kv((3, 7, 4, 32), "BLHc", 5)
    s0, _ = O.compute_qparams(x, "BLHc", "G_TOKEN_HEAD", 4)
    s1, z1 = O.compute_qparams(x, "BLHc", "G_TOKEN_HEAD", 4, symmetric=True, group_size=32)
    assert z1 is None and torch.equal(s0, s1)


def test_asymmetric_round_trip_error_bound():
    x = O.synthetic_kv((2, 9, 3, 64), "BLHc", 11)
    for bits in (2, 4, 8):
        for g in (None, 32, 16):
            s, z = O.compute_qparams(x, "BLHc", "G_TOKEN_HEAD", bits, symmetric=False, group_size=g, reduce_batch=False)
            codes = O.quantize(x, s, z, bits)
            lo, hi = O.bounds(bits)
            assert codes.min() >= lo and codes.max() <= hi
            assert torch.equal(z, torch.round(z)) and not torch.signbit(z[z == 0]).any()
            deq = O.dequantize(codes, s, z)
            err = (deq - x).abs()
            bound = O._per_element(s, 64) * 0.5001 + 1e-6
            # values inside the group's range are at most half a step away
            assert (err <= bound + O._per_element(s, 64) * 0.5).all()


def test_g_tensor_replace_semantics_differs_from_reference_defect():
    xs = [O.synthetic_kv((2, n, 3, 16), "BLHc", 70 + n) for n in (1, 4, 9)]
    a = O.OracleVARQ(8, "BLHc", "G_TENSOR", g_tensor_append_defect=True)
    b = O.OracleVARQ(8, "BLHc", "G_TENSOR", g_tensor_append_defect=False)
    for x in xs:
        a.use_var_q(x); b.use_var_q(x)
    assert a.cached_item.shape[1] == 21      # 1 -> 6 -> 21 tokens: duplicated
    assert b.cached_item.shape[1] == 14      # 1 + 4 + 9
