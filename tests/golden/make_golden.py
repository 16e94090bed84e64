"""Generate tests/golden/blockscaled_golden.npz from the reference's own host code.

Run where the reference tree is available (it builds oracle/_ref/libbsg_ref.so from the
reference headers): ``python tests/golden/make_golden.py``.  The vectors are outputs of
cutlass::reference::host::Gemm3x and of the reference's numeric types, on seeded inputs
that are stored alongside, so that the tests need neither the reference nor this script.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from cutlass_b200 import formats as F  # noqa: E402
from cutlass_b200 import generators as G  # noqa: E402


def main() -> None:
    oracle.build()
    ref = oracle.load_ref()
    if ref is None:
        raise SystemExit("reference driver not built (reference tree missing?)")
    out = {}
    # --- codecs: every code decoded, and a sweep of encodes
    for fmt, n in ((0, 16), (1, 256), (2, 256), (3, 256)):
        out[f"decode_{fmt}"] = np.array([ref.bsg_ref_decode(fmt, c) for c in range(n)], dtype=np.float32)
    rng = np.random.default_rng(2024)
    xs = [rng.standard_normal(400).astype(np.float32) * s for s in (1e-3, 0.05, 1.0, 8.0, 100.0, 600.0)]
    grid = np.array([0, 0.25, 0.5, 0.75, 1, 1.25, 1.5, 1.75, 2, 2.5, 3, 3.5, 4, 5, 6, 7, 448, 464, 480, 1e9,
                     2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -11, 2.0 ** -6, 0.0009765625, 17.0, 18.0, 19.0, 20.0, 22.0], dtype=np.float32)
    xs += [grid, -grid]
    # midpoints between neighbouring e4m3 values exercise the ties-to-even rule
    pos = F.decode_e4m3(np.arange(0x7F, dtype=np.uint8))
    xs.append(((pos[:-1].astype(np.float64) + pos[1:]) / 2).astype(np.float32))
    enc_in = np.concatenate(xs).astype(np.float32)
    out["encode_in"] = enc_in
    for fmt in (0, 1, 2, 3):
        out[f"encode_{fmt}"] = np.array([ref.bsg_ref_encode(fmt, float(x)) for x in enc_in], dtype=np.uint8)
    # e5m2 (an output type of the GEMM): every code decoded; encodes of the sweep above plus every midpoint between
    # neighbouring e5m2 values, their float32 neighbours, and the special values
    out["decode_4"] = np.array([ref.bsg_ref_decode(4, c) for c in range(256)], dtype=np.float32)
    pos5 = F.decode_e5m2(np.arange(0x7C, dtype=np.uint8))
    mid5 = ((pos5[:-1].astype(np.float64) + pos5[1:]) / 2).astype(np.float32)
    special = np.array([np.inf, -np.inf, np.nan, 57344.0, 61439.0, 61440.0, 65536.0, 1e9, -1e9, 0.0, -0.0], dtype=np.float32)
    enc5_in = np.concatenate([enc_in, mid5, -mid5, np.nextafter(mid5, np.float32(np.inf)), np.nextafter(mid5, np.float32(0)), special]).astype(np.float32)
    out["encode5_in"] = enc5_in
    out["encode_4"] = np.array([ref.bsg_ref_encode(4, float(x)) for x in enc5_in], dtype=np.uint8)
    # --- scale-factor layout
    for vec, rows, K in ((16, 300, 448), (32, 130, 1024), (16, 128, 64)):
        kb = F.ceil_div(K, vec)
        tab = np.array([[ref.bsg_ref_sf_offset(vec, rows, K, r, k * vec) for k in range(kb)] for r in range(rows)], dtype=np.int64)
        out[f"sf_offset_{vec}_{rows}_{K}"] = tab
        out[f"sf_size_{vec}_{rows}_{K}"] = np.array([ref.bsg_ref_sf_size(vec, rows, K)], dtype=np.int64)
    # --- GEMMs (fp32 and bf16 outputs) and the block-scaled output quantisation (NVFP4 and MXFP8)
    cases = [("nvfp4_a", 0, 96, 80, 128, 1.0, 0.5), ("nvfp4_b", 0, 130, 48, 320, 0.75, 0.0),
             ("mxfp8_a", 1, 96, 80, 128, 1.0, 0.5), ("mxfp8_b", 1, 40, 136, 96, -1.25, 2.0),
             ("mxfp4_a", 2, 72, 88, 256, 1.0, 0.5), ("mixed_a", 3, 100, 56, 384, 0.5, 1.0)]
    for name, kind, M, N, K, alpha, beta in cases:
        rng = np.random.default_rng(abs(hash(name)) % (2 ** 31))
        rng = np.random.default_rng(sum(ord(c) for c in name))
        gen_a, gen_b = G.operand_generators(kind, False)
        A, _, sfa = gen_a(M, K, rng)
        B, _, sfb = gen_b(N, K, rng)
        Cb = G.bf16_normal((M, N), rng)
        out[f"{name}_A"], out[f"{name}_B"], out[f"{name}_SFA"], out[f"{name}_SFB"], out[f"{name}_C"] = A, B, sfa, sfb, Cb
        out[f"{name}_dims"] = np.array([kind, M, N, K], dtype=np.int64)
        out[f"{name}_ab"] = np.array([alpha, beta], dtype=np.float32)
        out[f"{name}_D32"] = oracle.ref_gemm(kind, 0, A, sfa, B, sfb, M, N, K, Cb, alpha, beta)
        out[f"{name}_Dbf16"] = oracle.ref_gemm(kind, 1, A, sfa, B, sfb, M, N, K, Cb, alpha, beta)
        if kind >= 2:
            continue          # the general epilogue below is pinned on the two main kinds
        # the reference's general epilogue: act(alpha * acc + bias + beta * C), bias per column or per row
        bias_col, bias_row = (rng.standard_normal(n).astype(np.float32) * 3 for n in (N, M))
        out[f"{name}_bias_col"], out[f"{name}_bias_row"] = bias_col, bias_row
        for tag, bias, per_row, act in (("relu_col", bias_col, False, 1), ("gelu_col", bias_col, False, 2), ("silu_row", bias_row, True, 3)):
            out[f"{name}_D32_{tag}"] = oracle.ref_gemm_epi(kind, A, sfa, B, sfb, M, N, K, Cb, alpha, beta, bias, per_row, act)
    name, M, N, K = "quant_a", 70, 96, 192
    rng = np.random.default_rng(77)
    A, _, sfa = G.nvfp4_operand(M, K, rng)
    B, _, sfb = G.nvfp4_operand(N, K, rng)
    Cb = G.bf16_normal((M, N), rng)
    d32 = oracle.ref_gemm(0, 0, A, sfa, B, sfb, M, N, K, Cb, 1.0, 0.5)
    st = np.float32(448.0 * 6.0 / np.abs(d32).max())
    Dq, SFD = oracle.ref_gemm(0, 2, A, sfa, B, sfb, M, N, K, Cb, 1.0, 0.5, st)
    out.update({f"{name}_A": A, f"{name}_B": B, f"{name}_SFA": sfa, f"{name}_SFB": sfb, f"{name}_C": Cb,
                f"{name}_dims": np.array([0, M, N, K], dtype=np.int64), f"{name}_st": np.array([st], dtype=np.float32),
                f"{name}_D": Dq, f"{name}_SFD": SFD, f"{name}_D32": d32})
    # the same accumulators quantised to MXFP8 (e4m3 values, ue8m0 scale per 32, conversion rounds up)
    for tag, st_mx in (("mx1", np.float32(1.0)), ("mx2", np.float32(448.0 / np.abs(d32).max()))):
        Dm, SFm = oracle.ref_gemm(0, 3, A, sfa, B, sfb, M, N, K, Cb, 1.0, 0.5, st_mx)
        out.update({f"{name}_st_{tag}": np.array([st_mx], dtype=np.float32), f"{name}_D_{tag}": Dm, f"{name}_SFD_{tag}": SFm})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "blockscaled_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
