"""Generate the golden fixtures of this folder by running the reference itself.

Run once, in a container that has the reference checkout, as

    python tests/golden/make_golden.py --reference /path/to/VAR-Q

It imports the reference's ``VAR_Q.quant`` / ``VAR_Q.pack_unpack`` unmodified and
forces the pure-PyTorch packing path (the Triton wrappers assert CUDA tensors,
VAR_Q/pack_unpack.py:109,138, and VAR_Q/quant.py:3-8 binds only one backend), then
records what the reference produces on seeded inputs:

* ``pack_kat.json``      known-answer words for hand-written int8 rows;
* ``quant_small.npz``    inputs and, after every appended step, packed cache, scales and
                         the dequantised cache for 6 modes x 3 bit-widths x 2 layouts,
                         plus ragged head_dim and 16-bit input cases;
* ``quant_c1.json``      SHA-256 of codes / scales / dequantised output for the
                         [16,16,680,64] fp32 per-token-per-head INT4 case (too big to store).

The fixtures travel with the repository; the reference does not.
"""
import argparse
import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle.varq_oracle import MODES, synthetic_kv  # noqa: E402  (input generator only)

STEPS = (1, 4, 9, 16)


def load_reference(path):
    sys.path.insert(0, path)
    import VAR_Q.pack_unpack as P
    import VAR_Q.quant as Q
    Q._HAS_TRITON = False
    Q.pack_last_dim_to_int32_python = P.pack_last_dim_to_int32_python
    Q.unpack_last_dim_from_int32_python = P.unpack_last_dim_from_int32_python
    return Q, P


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def step_inputs(fmt, B, H, c, seed, dtype):
    out = []
    for i, n in enumerate(STEPS):
        shape = (B, n, H, c) if fmt == "BLHc" else (B, H, n, c)
        out.append(synthetic_kv(shape, fmt, seed * 100 + i, n_outlier=2, dtype=dtype))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (read-only)")
    args = ap.parse_args()
    Q, P = load_reference(args.reference)
    torch.set_num_threads(4)

    # ---- packing known answers
    rows = {
        "2": [[-2, 1, 0, -1] * 8],
        "4": [[-8, -5, -2, 1, 4, 7, -6, -3, 0, 3, 6, -7, -4, -1, 2, 5], [-8, 7, -1, 0, 3]],
        "8": [[-128, -125, -122, -119, -116, -113, -110, -107], [127, -1, 5]],
    }
    kat = []
    for bits, lst in rows.items():
        for r in lst:
            w, meta = P.pack_last_dim_to_int32_python(torch.tensor(r, dtype=torch.int8), int(bits))
            back = P.unpack_last_dim_from_int32_python(w, meta)
            assert back.tolist() == r
            kat.append({"bits": int(bits), "row": r, "words": [int(x) & 0xFFFFFFFF for x in w.tolist()], "meta": meta})
    # rounding / range behaviour of the quantizer (per-token-per-head groups)
    behav = []
    for bits, xs in ((4, [.5, 1.5, 2.5, -.5, -1.5, -2.5, 7, -7]), (2, [1, -1, .4, .6, -.5, .5, -2, 2]), (8, [0.0] * 8)):
        q = Q.VAR_Q(quant_bits=bits, qkv_format="BLHc", quant_method="G_TOKEN_HEAD")
        x = torch.tensor(xs, dtype=torch.float32).view(1, 1, 1, -1)
        q.quant(x)
        codes = P.unpack_last_dim_from_int32_python(q.quantized_item, q._pack_meta)
        behav.append({"bits": bits, "x": xs, "scale_bits": int(q.scale.view(-1).view(torch.int32)[0]),
                      "codes": codes.view(-1).tolist()})
    with open(os.path.join(HERE, "pack_kat.json"), "w") as f:
        json.dump({"pack": kat, "quant": behav}, f, indent=1)

    # ---- small multi-step sequences
    arrays, index = {}, []
    cases = [(fmt, mode, bits, 16, torch.float32) for fmt in ("BLHc", "BHLc") for mode in MODES for bits in (2, 4, 8)]
    cases += [("BLHc", "G_TOKEN_HEAD", 4, 20, torch.float32), ("BHLc", "G_SCALE_HEAD_DIM", 2, 20, torch.float32),
              ("BLHc", "G_SCALE_HEAD_DIM", 8, 16, torch.bfloat16), ("BHLc", "G_TOKEN_HEAD", 4, 16, torch.float16),
              ("BLHc", "G_TOKEN", 8, 5, torch.float32)]
    for ci, (fmt, mode, bits, c, dtype) in enumerate(cases):
        q = Q.VAR_Q(quant_bits=bits, qkv_format=fmt, quant_method=mode)
        xs = step_inputs(fmt, 2, 3, c, ci, dtype)
        key = f"case{ci}"
        index.append({"key": key, "fmt": fmt, "mode": mode, "bits": bits, "c": c,
                      "dtype": str(dtype).replace("torch.", ""), "steps": list(STEPS)})
        for si, x in enumerate(xs):
            out = q.use_var_q(x)
            arrays[f"{key}_x{si}"] = x.to(torch.float32).numpy()      # 16-bit inputs are exact in fp32
            arrays[f"{key}_codes{si}"] = q.cached_item.contiguous().numpy()
            arrays[f"{key}_scale{si}"] = q.cached_scale.contiguous().numpy()
            arrays[f"{key}_deq{si}"] = out.numpy()
    np.savez_compressed(os.path.join(HERE, "quant_small.npz"), **arrays)
    with open(os.path.join(HERE, "quant_small.json"), "w") as f:
        json.dump(index, f, indent=1)

    # ---- the [16,16,680,64] case, hashed
    x = synthetic_kv((16, 16, 680, 64), "BHLc", 0, n_outlier=4, dtype=torch.float32)
    q = Q.VAR_Q(quant_bits=4, qkv_format="BHLc", quant_method="G_TOKEN_HEAD")
    out = q.use_var_q(x)
    rec = {"shape": [16, 16, 680, 64], "fmt": "BHLc", "mode": "G_TOKEN_HEAD", "bits": 4, "seed": 0,
           "x_sha256": sha(x), "codes_sha256": sha(q.cached_item), "scale_sha256": sha(q.cached_scale),
           "deq_sha256": sha(out), "scale_shape": list(q.cached_scale.shape)}
    with open(os.path.join(HERE, "quant_c1.json"), "w") as f:
        json.dump(rec, f, indent=1)
    print("wrote fixtures:", len(kat), "pack KATs,", len(cases), "sequences, 1 hashed case")


if __name__ == "__main__":
    main()
