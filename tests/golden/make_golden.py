"""Regenerates the golden vectors in this directory from the REFERENCE's own host code.

Needs ``oracle/_ref/libref_host.so`` (built by ``make -C oracle ref`` from the reference
tree's headers).  The outputs are small and committed, so the tests can pin the oracle
and the operator mirror on machines where the reference tree is absent.

    python tests/golden/make_golden.py
"""
import ctypes
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))


class DespFields(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in
                ("dtype_a", "dtype_b", "dtype_c", "dacc", "dcomp", "trans_a", "trans_b", "trans_c")] + \
               [("tile_shape", ctypes.c_int * 3), ("warp_tile_shape", ctypes.c_int * 3),
                ("tensorop", ctypes.c_int * 3)] + \
               [(n, ctypes.c_int) for n in
                ("num_stage", "split_k_serial", "split_k_parallel", "shuffle_type", "epa_a", "epa_b", "epa_c",
                 "access_per_vector", "ndim", "op_type", "mask_sparse", "increment_k_first", "dynamic_mask",
                 "is_int8_inference")]


def desp_cases():
    """Descriptor field sets: the reference's own tile shapes for this path (Turing fp16 /
    int8 lists, cumm/gemm/main.py:462-524) and the sm_100a ones."""
    cases = []
    base = dict(dtype_a=7, dtype_b=7, dtype_c=7, dacc=0, dcomp=0, trans_a=0, trans_b=1, trans_c=0,
                tile_shape=[64, 64, 32], warp_tile_shape=[32, 32, 32], tensorop=[16, 8, 8], num_stage=2,
                split_k_serial=0, split_k_parallel=0, shuffle_type=0, epa_a=8, epa_b=8, epa_c=8,
                access_per_vector=1, ndim=3, op_type=0, mask_sparse=1, increment_k_first=1, dynamic_mask=0,
                is_int8_inference=0, algo="Turing")
    cases.append(dict(base))
    for op, (ta, tb) in ((0, (0, 1)), (1, (0, 0)), (2, (1, 0))):
        for ts, wts in (([64, 64, 32], [32, 32, 32]), ([128, 128, 32], [32, 64, 32]), ([128, 64, 32], [64, 32, 32]),
                        ([128, 128, 128], [128, 128, 128]), ([128, 64, 64], [128, 64, 64])):
            c = dict(base, op_type=op, trans_a=ta, trans_b=tb, tile_shape=ts, warp_tile_shape=wts,
                     split_k_serial=1 if op == 2 else 0)
            if ts[2] != 32:
                c.update(algo="Blackwell", tensorop=[128, ts[1], 16], num_stage=3)
            cases.append(c)
    cases.append(dict(base, dtype_a=3, dtype_b=3, dtype_c=3, dacc=1, dcomp=0, tensorop=[8, 8, 16], epa_a=16,
                      epa_b=16, epa_c=16, is_int8_inference=1))
    cases.append(dict(base, dynamic_mask=1, increment_k_first=0))
    for sh in (1, 2):
        cases.append(dict(base, shuffle_type=sh, trans_a=1 if sh == 2 else 0, trans_b=0 if sh == 2 else 1,
                          split_k_serial=1 if sh == 2 else 0, algo="Turing"))
    cases.append(dict(base, algo="Simt", tensorop=[-1, -1, -1], tile_shape=[32, 64, 8], warp_tile_shape=[32, 32, 8],
                      dtype_a=0, dtype_b=0, dtype_c=0, epa_a=1, epa_b=1, epa_c=1, mask_sparse=0))
    cases.append(dict(base, split_k_parallel=1, split_k_serial=0))
    return cases


def to_struct(c):
    f = DespFields()
    for k, v in c.items():
        if k == "algo":
            continue
        if isinstance(v, list):
            setattr(f, k, (ctypes.c_int * 3)(*v))
        else:
            setattr(f, k, v)
    return f


def main():
    R = ctypes.CDLL(str(ROOT / "oracle" / "_ref" / "libref_host.so"))
    R.ref_float_to_half.restype = ctypes.c_uint16
    R.ref_float_to_half.argtypes = [ctypes.c_float]
    R.ref_half_to_float.restype = ctypes.c_float
    R.ref_half_to_float.argtypes = [ctypes.c_uint16]
    R.ref_float_to_s8.restype = ctypes.c_int
    R.ref_float_to_s8.argtypes = [ctypes.c_float]

    rng = np.random.default_rng(20240607)
    # ---- fp32 -> fp16: random magnitudes over the whole half range, ties, subnormals, specials
    vals = [0.0, -0.0, 1.0, -1.0, 0.1, 65504.0, 65519.9, 65520.0, 65536.0, 1e-8, 5.9604645e-08, 2.9802322e-08,
            2.98023224e-08 * 1.0000001, 6.1035156e-05, 6.0975552e-05, 1e-30, float("inf"), -float("inf")]
    vals += list((rng.standard_normal(1500) * np.exp(rng.uniform(-20, 12, 1500))).astype(np.float32))
    # exact ties between adjacent halves
    for h in rng.integers(0, 0x7BFF, 400):
        lo = R.ref_half_to_float(int(h))
        hi = R.ref_half_to_float(int(h) + 1)
        vals.append((lo + hi) / 2)
        vals.append(-(lo + hi) / 2)
    f = np.array(vals, np.float32)
    h = np.array([R.ref_float_to_half(float(v)) for v in f], np.uint16)
    # ---- fp16 -> fp32: every finite half and the infinities
    allh = np.array([b for b in range(65536) if (b & 0x7C00) != 0x7C00 or (b & 0x3FF) == 0], np.uint16)
    allf = np.array([R.ref_half_to_float(int(b)) for b in allh], np.float32)
    # ---- fp32 -> int8 (within int32 range: beyond it the reference's HOST twin is undefined)
    s = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, 127.5, 128.5, -127.5, -128.5, -129.5, 200.0, -300.0, 1e6, -1e6,
         0.49999997, -0.49999997, 1e-9]
    s += list((rng.standard_normal(1500) * 60).astype(np.float32))
    s += list((rng.integers(-140, 140, 300) + 0.5).astype(np.float32))
    s = np.array(s, np.float32)
    q = np.array([R.ref_float_to_s8(float(v)) for v in s], np.int8)
    np.savez_compressed(HERE / "numerics.npz", f32_to_f16_in=f, f32_to_f16_out=h, f16_bits=allh, f16_to_f32=allf,
                        f32_to_s8_in=s, f32_to_s8_out=q)

    # ---- contract arithmetic
    recs = []
    buf = ctypes.create_string_buffer(512)
    for c in desp_cases():
        st = to_struct(c)
        algo = c["algo"].encode()
        rec = dict(fields=c)
        rc = R.ref_gemm_desp_repr(ctypes.byref(st), algo, buf, 512)
        rec["gemm_repr"] = buf.value.decode() if rc == 0 else None
        rc = R.ref_conv_desp_repr(ctypes.byref(st), algo, buf, 512)
        rec["conv_repr"] = buf.value.decode() if rc == 0 else None
        probes = []
        for (N, C, K, kv, mw, sk) in ((150000, 128, 128, 27, 128, 32), (150000, 64, 64, 27, 64, 1),
                                       (491092, 128, 128, 27, 128, 8), (1000, 24, 40, 27, 96, 4),
                                       (777, 130, 64, 8, 32, 2)):
            mnk = (ctypes.c_int * 3)()
            R.ref_implicit_gemm_mnk(c["op_type"], N, C, K, kv, mnk)
            m, n, k = list(mnk)
            tc = (ctypes.c_int * 3)()
            R.ref_spconv_tile_count(m, n, k, c["tile_shape"][0], c["tile_shape"][1], sk, kv, c["op_type"], tc)
            pr = dict(N=N, C=C, K=K, kv=kv, mask_width=mw, split_k=sk, mnk=[m, n, k], tiles=list(tc),
                      gemm_supported=R.ref_gemm_desp_supported(ctypes.byref(st), m, n, k),
                      conv_supported=R.ref_conv_desp_supported(ctypes.byref(st), m, n, k, C, K, mw),
                      k_per_split=R.ref_gemm_k_size_per_split(k, sk, c["tile_shape"][2]))
            if sk == 1 or c["split_k_serial"] or c["split_k_parallel"]:
                pr["gemm_workspace"] = R.ref_gemm_workspace(ctypes.byref(st), m, n, k, sk)
                pr["conv_workspace"] = R.ref_conv_workspace(ctypes.byref(st), m, n, k, sk, kv)
            probes.append(pr)
        rec["probes"] = probes
        recs.append(rec)
    (HERE / "contract.json").write_text(json.dumps(recs, indent=1))
    print("wrote", HERE / "numerics.npz", HERE / "contract.json", len(f), len(s), len(recs))


if __name__ == "__main__":
    main()
