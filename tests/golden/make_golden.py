"""Writes tests/golden/golden.json from the installed PyTorch's CPU kernels.

Run from the repository root: python tests/golden/make_golden.py

The reference stores no golden vectors (its tests compute expectations from
seeded generators against PyTorch's CPU, tests/python/test_quant.py); these
fixtures freeze those CPU results for the same seeded cases: SHA-256 of the
dyn-int4 packed weights and outputs (bit-exact ops), and the leading outputs of
the int8 and float8 products (compared within the reference's error bound).
"""

import hashlib
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import _cases as C  # noqa: E402


def digest(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def main():
    out = {"torch": torch.__version__, "dyn4": [], "int8": [], "fp8": []}
    for (m, k, n, bs, bias) in C.DYN4_CASES:
        for dtype in (torch.float32, torch.bfloat16):
            if dtype == torch.bfloat16 and bs != k:
                continue
            x, w, sc, bvec = C.dyn4_case(m, k, n, bs, bias, dtype)
            packed = torch._dyn_quant_pack_4bit_weight(w, sc, bvec, bs, k, n)
            res = torch._dyn_quant_matmul_4bit(x, packed, bs, k, n)
            out["dyn4"].append({"shape": [m, k, n, bs, bias], "dtype": str(dtype).split(".")[1],
                                "packed_sha256": digest(packed), "out_sha256": digest(res),
                                "out_head": res.reshape(-1)[:8].float().tolist()})
    for (m, k, n) in C.INT8_SHAPES:
        for dtype in C.INT8_DTYPES:
            a, b, s = C.int8_case(dtype, m, k, n)
            want, _ = C.int8_want(a, b, s)
            out["int8"].append({"shape": [m, k, n], "dtype": str(dtype).split(".")[1],
                                "out_head": want.reshape(-1)[:16].float().tolist()})
    for fa, fb in ((C.FLOAT8[0], C.FLOAT8[0]), (C.FLOAT8[1], C.FLOAT8[0]), (C.FLOAT8[0], C.FLOAT8[1])):
        for od in (torch.bfloat16, torch.float32, torch.float16, torch.float8_e4m3fn, None):
            for rowwise in (False, True):
                a, b, sa, sb, bias, sr = C.scaled_case(fa, fb, od, rowwise)
                want, _ = C.scaled_want(a, b, sa, sb, bias, sr, od)
                out["fp8"].append({"fa": str(fa).split(".")[1], "fb": str(fb).split(".")[1],
                                   "out_dtype": str(od).split(".")[1] if od else None, "rowwise": rowwise,
                                   "out_head": want.reshape(-1)[:16].float().tolist()})
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", len(out["dyn4"]), len(out["int8"]), len(out["fp8"]), "cases")


if __name__ == "__main__":
    main()
