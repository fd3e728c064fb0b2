"""Regenerates tests/golden/golden_v1.npz from the CPU oracle.

The reference stores no golden vectors and its array library (mlx) cannot be
imported where this repository is built, so these fixtures freeze the oracle's
own outputs on seeded inputs: they guard the oracle against accidental change
and give the GPU tests byte-level expectations that do not depend on running
the oracle.  Run from the repository root:  python tests/golden/make_golden.py
"""

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import tq_oracle as o  # noqa: E402


def main():
    rng = np.random.default_rng(20240607)
    out = {}
    d = 128
    s42, s43 = o.signs_from_seed(d, 42), o.signs_from_seed(d, 43)
    out["signs_42"], out["signs_43"] = s42, s43
    out["signs64_42"] = o.signs_from_seed(64, 42)
    x = (rng.standard_normal((96, d)) * rng.lognormal(0.0, 0.5, (96, 1))).astype(np.float16)
    x[0] = 0                      # zero vector
    x[1] = s43.astype(np.float16)  # x == signs
    out["x_f16"] = x
    for bits in (1, 2, 3, 4):
        p, n = o.quantize_packed(x, s43, bits)
        out[f"packed_b{bits}"] = p
        out[f"deq_b{bits}"] = o.packed_dequantize(p, n, o.codebook(bits), s43, d, bits)
    out["norms"] = n
    x64 = rng.standard_normal((40, 64)).astype(np.float32)
    out["x64_f32"] = x64
    p64, n64 = o.quantize_packed(x64, out["signs64_42"], 4)
    out["packed64_b4"], out["norms64"] = p64, n64

    # decode attention, dense fp16 K + 3-bit V (GQA 2 kv heads x 7)
    n_kv, n_rep, S = 2, 7, 160
    kd = rng.standard_normal((n_kv, S, d)).astype(np.float16)
    vraw = (rng.standard_normal((n_kv, S, d)) * rng.lognormal(0.0, 0.5, (n_kv, S, 1))).astype(np.float16)
    q = rng.standard_normal((n_kv * n_rep, d)).astype(np.float16)
    vp, vn = o.quantize_packed(vraw, s43, 3)
    scale = 1.0 / np.sqrt(d)
    vdesc = dict(packed=vp, norms=vn, centroids=o.codebook(3), signs=s43, bits=3)
    att, _ = o.decode_attention(q, k_dense=kd, v_polar=vdesc, attn_scale=scale, n_rep=n_rep)
    out.update(att_q=q, att_kd=kd, att_vp=vp, att_vn=vn, att_out_dense=att)
    # polar 4-bit K + 3-bit V
    kraw = (rng.standard_normal((n_kv, S, d)) * rng.lognormal(0.0, 0.5, (n_kv, S, 1))).astype(np.float16)
    kp, kn = o.quantize_packed(kraw, s42, 4)
    kdesc = dict(packed=kp, norms=kn, centroids=o.codebook(4), signs=s42, bits=4)
    att2, _ = o.decode_attention(q, k_polar=kdesc, v_polar=vdesc, attn_scale=scale, n_rep=n_rep)
    out.update(att_kp=kp, att_kn=kn, att_out_polar=att2)
    out["q_rot"] = o.prerotate_query(q, s42)
    out["scores_polar"] = o.prerot_fused_qk_scores(out["q_rot"], kp, kn, o.codebook(4), d, 4, n_rep)
    np.savez_compressed(os.path.join(HERE, "golden_v1.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
