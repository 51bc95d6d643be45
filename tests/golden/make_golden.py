"""Regenerates tests/golden/golden.npz from the REFERENCE's own host code.

Run where the reference tree is present and `make -C oracle ref` has built
oracle/_ref/libw4ref.so:

    python tests/golden/make_golden.py

For every (shape, seed) case of the reference's gates (tests/cases.py) the file
stores sha256 digests of the bitwise artefacts the reference produced (packed
codes, scales, zeros, dequantised FP16) and the reference's FP64 GEMM /
attention outputs in full. The oracle and the CUDA path are then checked
against these vectors on machines that do not have the reference.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import cases  # noqa: E402
from oracle import orc  # noqa: E402


def main():
    r = orc.Reference()
    g = {}
    for sym in (True, False):
        for i, (M, N, K, gs) in enumerate(cases.GEMM_CFGS):
            seed = cases.w4_seed(i, sym)
            w = r.normal_f64(N * K, seed)
            x = r.normal_f16(M * K, seed + 1)
            p = r.quantize_w4(w, N, K, gs, sym)
            wd = r.dequant_all_w4(p)
            key = f"w4/{'sym' if sym else 'asym'}/{i}"
            g[key + "/packed"] = np.array(cases.digest(p["q"], p["scales"], p["zeros"]))
            g[key + "/dequant"] = np.array(cases.digest(wd))
            g[key + "/x"] = np.array(cases.digest(x))
            g[key + "/c"] = r.gemm_oracle(x, M, K, wd, N)
    for i, (M, N, K) in enumerate(cases.MX_HOST_CFGS):
        w = r.normal_f64(N * K, cases.mx_host_seed(i))
        p = r.quantize_mx(w, N, K)
        g[f"mxhost/{i}/packed"] = np.array(cases.digest(p["q"], p["scales"]))
        g[f"mxhost/{i}/dequant"] = np.array(cases.digest(r.dequant_all_mx(p)))
    for i, (M, N, K, _) in enumerate(cases.GEMM_CFGS):
        seed = cases.mx_gpu_seed(i)
        w = r.normal_f64(N * K, seed)
        x = r.normal_f16(M * K, seed + 1)
        p = r.quantize_mx(w, N, K)
        wd = r.dequant_all_mx(p)
        g[f"mx/{i}/packed"] = np.array(cases.digest(p["q"], p["scales"]))
        g[f"mx/{i}/dequant"] = np.array(cases.digest(wd))
        g[f"mx/{i}/c"] = r.gemm_oracle(x, M, K, wd, N)
    for sym in (True, False):
        for name, cfgs, seedf in (("kv", cases.KV_CFGS, cases.kv_seed), ("kvlong", cases.KV_LONG_CFGS, cases.kv_long_seed)):
            for i, (H, S, D, gs) in enumerate(cfgs):
                seed = seedf(i, sym)
                k = r.normal_f64(H * S * D, seed)
                v = r.normal_f64(H * S * D, seed + 1)
                q = r.normal_f16(H * D, seed + 2)
                c = r.quantize_cache_w4(k, v, H, S, D, gs, sym)
                out, kd, vd = r.attention_w4(q, c)
                key = f"{name}/{'sym' if sym else 'asym'}/{i}"
                g[key + "/packed"] = np.array(cases.digest(c["q_k"], c["s_k"], c["z_k"], c["q_v"], c["s_v"], c["z_v"]))
                g[key + "/dequant"] = np.array(cases.digest(kd, vd))
                g[key + "/out"] = out
    for i, (H, S, D, gs) in enumerate(cases.KV_CFGS + [cases.KV_LONG_CFGS[1]]):
        seed = cases.f8_gpu_seed(i)
        k = r.normal_f64(H * S * D, seed)
        v = r.normal_f64(H * S * D, seed + 1)
        q = r.normal_f16(H * D, seed + 2)
        c = r.quantize_cache_f8(k, v, H, S, D, gs)
        out, kd, vd = r.attention_f8(q, c)
        g[f"f8/{i}/packed"] = np.array(cases.digest(c["q_k"], c["s_k"], c["q_v"], c["s_v"]))
        g[f"f8/{i}/dequant"] = np.array(cases.digest(kd, vd))
        g[f"f8/{i}/out"] = out
    for sym in (True, False):
        for i, (H, S, D, gs, page) in enumerate(cases.PAGED_CFGS):
            seed = cases.paged_seed(i, sym)
            k = r.normal_f64(H * S * D, seed)
            v = r.normal_f64(H * S * D, seed + 1)
            c = r.quantize_cache_w4(k, v, H, S, D, gs, sym)
            lp = (S + page - 1) // page
            bt = np.random.default_rng(seed ^ 0x5ED).permutation(lp).astype(np.int32)
            p = r.paged_from_contiguous(c, page, bt)
            g[f"paged/{'sym' if sym else 'asym'}/{i}/pool"] = np.array(
                cases.digest(p["q_k"], p["s_k"], p["z_k"], p["q_v"], p["s_v"], p["z_v"]))
    np.savez_compressed(os.path.join(HERE, "golden.npz"), **g)
    print("wrote", len(g), "entries,", os.path.getsize(os.path.join(HERE, "golden.npz")), "bytes")


if __name__ == "__main__":
    main()
