#!/usr/bin/env python3
"""Runs the reference's own x86 kernels on seeded inputs and writes their outputs.

The reference's model code is Rust and cannot be compiled here, but its hottest kernels are
plain assembly files that gcc assembles as they are.  This script assembles, read-only from the
reference's source tree (first argument, or $HERBERT_RS_SOURCE),

    crates/backends/backend_bf16_avx512/src/avx512_bf16_matvec.S      avx512_bf16_matvec_tile
    crates/backends/backend_common/src/avx512_attn_dot8_bf16.S        avx512_attn_dot8_qf32_kbf16
    crates/backends/backend_common/src/avx512_fused_attn_bf16.S       avx512_fused_attn_step8_bf16
    crates/backends/backend_common/src/avx512_softmax_8head.S         avx512_softmax_8head_inplace
    crates/backends/backend_common/src/avx512_2pass_sv_bf16.S         avx512_2pass_sv8_bf16

into a shared library in a temporary folder, calls them through ctypes as the reference's Rust
code does (crates/backends/backend_common/src/generic_attention/ffi.rs:3-113;
prefill/kernel_bf16.rs:150-300 for the order of calls, the initial m = -inf, l = 0 and the final
division by l), and stores inputs' seeds and the kernels' outputs in
`reference_kernels_golden.npz` beside this file.  It needs a CPU with AVX-512 BF16.

    python tests/golden/make_reference_kernels_golden.py /path/to/herbert-rs

`tests/test_reference_anchor.py` compares the plain implementation with the stored outputs, and,
where the reference's sources, gcc and such a CPU are at hand, runs this script's `run_kernels`
again and checks that the stored outputs are what the kernels give.
"""
import ctypes
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "reference_kernels_golden.npz")
SOURCES = ["backend_bf16_avx512/src/avx512_bf16_matvec.S", "backend_common/src/avx512_attn_dot8_bf16.S",
           "backend_common/src/avx512_fused_attn_bf16.S", "backend_common/src/avx512_softmax_8head.S",
           "backend_common/src/avx512_2pass_sv_bf16.S"]
# sizes: a product with K no multiple of 32 and N no multiple of 4; attention with head sizes 128 and 64
MATVEC = dict(seed=101, N=37, K=200)
ATTN = [dict(seed=202, hd=128, keys=77), dict(seed=203, hd=64, keys=130)]


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns, round to nearest even (crates/core/src/tensor.rs:46-56)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def inputs():
    """The seeded inputs, as the test rebuilds them too."""
    out = {}
    r = np.random.default_rng(MATVEC["seed"])
    out["matvec_x"] = r.standard_normal(MATVEC["K"]).astype(np.float32)
    out["matvec_w"] = to_bf16_bits(r.standard_normal((MATVEC["N"], MATVEC["K"])).astype(np.float32) * 0.1)
    for i, a in enumerate(ATTN):
        r = np.random.default_rng(a["seed"])
        out[f"attn{i}_q"] = r.standard_normal((8, a["hd"])).astype(np.float32)            # 8 query heads of one kv head
        out[f"attn{i}_k"] = to_bf16_bits(r.standard_normal((a["keys"], a["hd"])).astype(np.float32))
        out[f"attn{i}_v"] = to_bf16_bits(r.standard_normal((a["keys"], a["hd"])).astype(np.float32))
    return out


def build(source_root: str, out_dir: str) -> ctypes.CDLL:
    base = os.path.join(source_root, "crates", "backends")
    lib = os.path.join(out_dir, "libreference_kernels.so")
    cmd = ["gcc", "-shared", "-fPIC", "-Wl,-z,noexecstack", "-o", lib] + [os.path.join(base, s) for s in SOURCES] + \
          ["-I", os.path.join(base, "backend_common", "src")]
    subprocess.run(cmd, check=True, stdout=subprocess.PIPE, stderr=subprocess.PIPE)
    return ctypes.CDLL(lib)


def run_kernels(source_root: str) -> dict:
    f32p, u16p = ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_uint16)
    ptr = lambda a, t: a.ctypes.data_as(t)
    inp, out = inputs(), {}
    with tempfile.TemporaryDirectory() as d:
        lib = build(source_root, d)
        # y = W bf16(x)
        x, w = inp["matvec_x"], np.ascontiguousarray(inp["matvec_w"])
        y = np.zeros(MATVEC["N"], dtype=np.float32)
        lib.avx512_bf16_matvec_tile.argtypes = [f32p, u16p, f32p, ctypes.c_uint64, ctypes.c_uint64]
        lib.avx512_bf16_matvec_tile.restype = None
        lib.avx512_bf16_matvec_tile(ptr(x, f32p), ptr(w, u16p), ptr(y, f32p), MATVEC["N"], MATVEC["K"])
        out["matvec_y"] = y
        lib.avx512_attn_dot8_qf32_kbf16.argtypes = [ctypes.POINTER(f32p), u16p, ctypes.c_uint64, f32p]
        lib.avx512_attn_dot8_qf32_kbf16.restype = None
        lib.avx512_fused_attn_step8_bf16.argtypes = [ctypes.POINTER(f32p), u16p, u16p, f32p, f32p, ctypes.c_uint64, ctypes.c_float]
        lib.avx512_fused_attn_step8_bf16.restype = None
        lib.avx512_softmax_8head_inplace.argtypes = [f32p, ctypes.c_uint64]
        lib.avx512_softmax_8head_inplace.restype = None
        lib.avx512_2pass_sv8_bf16.argtypes = [f32p, u16p, f32p, ctypes.c_uint64, ctypes.c_uint64]
        lib.avx512_2pass_sv8_bf16.restype = None
        for i, a in enumerate(ATTN):
            hd, n = a["hd"], a["keys"]
            q = np.ascontiguousarray(inp[f"attn{i}_q"])
            k, v = np.ascontiguousarray(inp[f"attn{i}_k"]), np.ascontiguousarray(inp[f"attn{i}_v"])
            qp = (f32p * 8)(*[ptr(q[h], f32p) for h in range(8)])
            scale = np.float32(1.0 / np.sqrt(hd))
            # raw dot products of the 8 heads with every key: scores[j*8 + h]
            scores = np.zeros((n, 8), dtype=np.float32)
            for j in range(n):
                lib.avx512_attn_dot8_qf32_kbf16(qp, ptr(k[j], u16p), hd, ptr(scores[j], f32p))
            out[f"attn{i}_dots"] = scores.copy()
            # online softmax, one key per call: o, (m, l) carried between calls; then o / l
            o = np.zeros((8, hd), dtype=np.float32)
            ml = np.concatenate([np.full(8, -np.inf, dtype=np.float32), np.zeros(8, dtype=np.float32)])
            for j in range(n):
                lib.avx512_fused_attn_step8_bf16(qp, ptr(k[j], u16p), ptr(v[j], u16p), ptr(o, f32p), ptr(ml, f32p), hd, scale)
            out[f"attn{i}_online"] = o / ml[8:, None]
            out[f"attn{i}_m"] = ml[:8].copy()
            # the two-pass path: scaled scores -> softmax in place -> weighted sum of v
            s2 = np.ascontiguousarray(scores * scale)
            lib.avx512_softmax_8head_inplace(ptr(s2, f32p), n)
            out[f"attn{i}_probs"] = s2.copy()
            o2 = np.zeros((8, hd), dtype=np.float32)
            lib.avx512_2pass_sv8_bf16(ptr(s2, f32p), ptr(v, u16p), ptr(o2, f32p), hd, n)
            out[f"attn{i}_twopass"] = o2
    return out


def main() -> int:
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("HERBERT_RS_SOURCE")
    if not root:
        print("usage: make_reference_kernels_golden.py /path/to/herbert-rs", file=sys.stderr)
        return 2
    np.savez(GOLDEN, **run_kernels(root))
    print(f"wrote {GOLDEN}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
