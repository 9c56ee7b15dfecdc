"""Regenerates the golden fixtures in this directory from the reference's own example generators.

Run in a checkout that has the asc-devkit tree available (pass its path with --reference):

    python tests/golden/make_golden.py [--reference /path/to/asc-devkit]

Each reference ``scripts/gen_data.py`` is executed unmodified (runpy, in a scratch directory, numpy's global
seed fixed first) and the ``input/*.bin`` / ``output/golden.bin`` files it writes are collected into one
``.npz`` per example.  The fixtures are what the oracle is pinned against; the tests never need the reference
tree itself.
"""
import argparse
import os
import runpy
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
EX = "examples/01_simd_cpp_api/04_advanced_api/03_quantization"
KEEP_ROWS = 96

# (fixture name, script, argv, seed, {bin file: (dtype, shape)})
CASES = [
    ("quant_dav2201", f"{EX}/quant/scripts/gen_data.py", ["dav-2201"], 101,
     {"input/input.bin": (np.float32, (1024,)), "output/golden.bin": (np.int8, (1024,))}),
    ("quant_dav3510", f"{EX}/quant/scripts/gen_data.py", ["dav-3510"], 102,
     {"input/input.bin": (np.float32, (1024,)), "output/golden.bin": (np.int8, (1024,))}),
    ("dequant", f"{EX}/dequant/scripts/gen_data.py", [], 103,
     {"input/input.bin": (np.int32, (128, 32)), "input/scale.bin": (np.float32, (32,)),
      "output/golden.bin": (np.float32, (128, 32))}),
    ("antiquant_dav2201", f"{EX}/antiquant/scripts/gen_data.py", ["dav-2201"], None,
     {"input/input_src.bin": (np.int8, (8, 128)), "input/input_offset.bin": (np.float16, (1, 128)),
      "input/input_scale.bin": (np.float16, (1, 128)), "output/golden.bin": (np.float16, (8, 128))}),
    ("matmul_quant_scalar", "examples/01_simd_cpp_api/04_advanced_api/00_matmul/matmul_quant/scripts/gen_data.py", ["-m", "0"], 104,
     {"input/x1_gm.bin": (np.int8, (1024, 1024)), "input/x2_gm.bin": (np.int8, (1024, 1024)),
      "input/bias_gm.bin": (np.int32, (1024,)), "output/golden.bin": (np.float16, (1024, 1024))}),
    ("matmul_quant_vector", "examples/01_simd_cpp_api/04_advanced_api/00_matmul/matmul_quant/scripts/gen_data.py", ["-m", "1"], 105,
     {"input/x1_gm.bin": (np.int8, (1024, 1024)), "input/x2_gm.bin": (np.int8, (1024, 1024)),
      "input/bias_gm.bin": (np.int32, (1024,)), "input/quant_vector_gm.bin": (np.uint64, (1024,)),
      "output/golden.bin": (np.float16, (1024, 1024))}),
    ("matmul_mx_e5m2", "examples/01_simd_cpp_api/04_advanced_api/00_matmul/matmul_mx/scripts/gen_data.py", [], 106,
     {"input/x1_gm.bin": (np.uint8, (32, 128)), "input/x2_gm.bin": (np.uint8, (128, 128)),
      "input/x1_mx_gm.bin": (np.uint8, (32, 4)), "input/x2_mx_gm.bin": (np.uint8, (2, 128, 2)),
      "output/golden.bin": (np.float32, (32, 128))}),
    ("mmad_mx_scenario3", "examples/01_simd_cpp_api/03_basic_api/03_matrix_compute/mmad_mx/scripts/gen_data.py",
     ["scenario_num=3"], 107,
     {"input/x1_gm.bin": (np.uint8, (40, 70)), "input/x2_gm.bin": (np.uint8, (50, 70)),
      "input/x1_scale_gm.bin": (np.uint8, (40, 4)), "input/x2_scale_gm.bin": (np.uint8, (50, 4)),
      "output/golden.bin": (np.float32, (40, 50))}),
    ("mmad_mx_scenario4", "examples/01_simd_cpp_api/03_basic_api/03_matrix_compute/mmad_mx/scripts/gen_data.py",
     ["scenario_num=4"], 108,
     {"input/x1_gm.bin": (np.uint8, (40, 70)), "input/x2_gm.bin": (np.uint8, (50, 70)),
      "input/x1_scale_gm.bin": (np.uint8, (40, 4)), "input/x2_scale_gm.bin": (np.uint8, (50, 4)),
      "input/bias_gm.bin": (np.float32, (50,)), "output/golden.bin": (np.float32, (40, 50))}),
    ("antiquant_dav3510", f"{EX}/antiquant/scripts/gen_data.py", ["dav-3510"], None,
     {"input/input_src.bin": (np.int8, (8, 128)), "input/input_offset.bin": (np.float16, (1, 128)),
      "input/input_scale.bin": (np.float16, (1, 128)), "output/golden.bin": (np.float16, (8, 128))}),
]


FIXPIPE = "examples/01_simd_cpp_api/03_basic_api/03_matrix_compute/fixpipe_l0c2gm/scripts/gen_data_s322s8.py"


def fixpipe_req8(reference):
    """The fixpipe sample's int32 -> int8 generator has no command line: its functions are called directly.  Two
    fixtures: the sample's own matmul case (vector parameters, no ReLU, row-major output), and its scalar routine
    ``req8_pre`` on single values that exercise rounding, the offset, both result types and the shift mode."""
    path = os.path.join(reference, FIXPIPE)
    with tempfile.TemporaryDirectory() as tmp:
        cwd = os.getcwd()
        os.chdir(tmp)
        try:
            mod = runpy.run_path(path)          # seeds numpy's global generator with 9
            mod["gen_golden_data"](1, 2, 0)
            x1 = np.fromfile("input/x1_gm.bin", np.int8).reshape(2, 128, 64).transpose(1, 0, 2).reshape(128, 128)
            out = {"x1_gm": np.ascontiguousarray(x1),
                   "x2_gm": np.fromfile("input/x2_gm.bin", np.int8).reshape(128, 256),
                   "quant_pre": np.fromfile("input/quant_pre.bin", np.uint64),
                   "golden": np.fromfile("output/golden.bin", np.int8).reshape(128, 256)}
        finally:
            os.chdir(cwd)
    np.savez_compressed(os.path.join(HERE, "fixpipe_req8_matmul.npz"), **out)
    print("fixpipe_req8_matmul", {k: v.shape for k, v in out.items()})

    rng = np.random.default_rng(109)
    n = 6000
    scale = rng.uniform(0.0005, 3.0, n).astype(np.float32) * rng.choice([1.0, 1.0, 1.0, -1.0], n).astype(np.float32)
    scale[:64] = rng.choice([0.5, 0.25, 1.5, 2.0, 0.125], 64).astype(np.float32)        # products that land on .5 ties
    bits = scale.view(np.uint32).astype(np.uint64)
    bits[64:96] = rng.integers(0, 1 << 23, 32).astype(np.uint64)                           # zero exponent field
    data = np.where(rng.random(n) < 0.5, rng.integers(-600, 600, n), rng.integers(-(1 << 31), 1 << 31, n)).astype(np.int32)
    data[:64] = rng.integers(-511, 511, 64)
    offset = np.where(rng.random(n) < 0.4, 0, rng.integers(0, 512, n)).astype(np.uint64)
    sign = rng.integers(0, 2, n).astype(np.uint64)
    mcb = (rng.random(n) < 0.3).astype(np.uint64)
    shift = rng.integers(0, 16, n).astype(np.uint64)
    q = bits | (shift << np.uint64(32)) | (mcb << np.uint64(36)) | (offset << np.uint64(37)) | (sign << np.uint64(46))
    req8 = mod["req8_pre"]
    with np.errstate(all="ignore"):
        res = np.array([int(req8(np.int32(d), int(w), int(w) & 0xFFFFFFFF)) for d, w in zip(data, q)], np.int16)
    np.savez_compressed(os.path.join(HERE, "fixpipe_req8_values.npz"), data=data, quant_pre=q, golden=res)
    print("fixpipe_req8_values", n)


def fixpipe_qf322b8(reference):
    """The same for the sample's fp32 -> int8 generator (half operands, fp32 accumulator): its matmul case, and its
    scalar routine ``qf322b8_pre`` on single values (shift mode off: the field table says it does not apply here)."""
    path = os.path.join(reference, os.path.dirname(FIXPIPE), "gen_data_f322s8.py")
    with tempfile.TemporaryDirectory() as tmp:
        cwd = os.getcwd()
        os.chdir(tmp)
        try:
            mod = runpy.run_path(path)
            mod["gen_golden_data"](1, 2, 0)
            x1 = np.fromfile("input/x1_gm.bin", np.float16).reshape(2, 128, 64).transpose(1, 0, 2).reshape(128, 128)
            out = {"x1_gm": np.ascontiguousarray(x1),
                   "x2_gm": np.fromfile("input/x2_gm.bin", np.float16).reshape(128, 256),
                   "quant_pre": np.fromfile("input/quant_pre.bin", np.uint64),
                   "golden": np.fromfile("output/golden.bin", np.int8).reshape(128, 256)}
        finally:
            os.chdir(cwd)
    np.savez_compressed(os.path.join(HERE, "fixpipe_qf322b8_matmul.npz"), **out)
    print("fixpipe_qf322b8_matmul", {k: v.shape for k, v in out.items()})

    rng = np.random.default_rng(110)
    n = 6000
    scale = rng.uniform(0.0005, 3.0, n).astype(np.float32) * rng.choice([1.0, 1.0, 1.0, -1.0], n).astype(np.float32)
    scale[:64] = rng.choice([0.5, 0.25, 1.5, 2.0, 0.125], 64).astype(np.float32)
    bits = scale.view(np.uint32).astype(np.uint64)
    data = np.where(rng.random(n) < 0.6, rng.uniform(-400, 400, n), rng.normal(0, 1e6, n)).astype(np.float32)
    data[:64] = rng.integers(-511, 511, 64).astype(np.float32)          # with the scales above: exact .5 ties
    offset = np.where(rng.random(n) < 0.4, 0, rng.integers(0, 512, n)).astype(np.uint64)
    sign = rng.integers(0, 2, n).astype(np.uint64)
    q = bits | (offset << np.uint64(37)) | (sign << np.uint64(46))
    fn = mod["qf322b8_pre"]
    with np.errstate(all="ignore"):
        res = np.array([int(fn(np.float32(d), int(w), int(w) & 0xFFFFFFFF)) for d, w in zip(data, q)], np.int16)
    np.savez_compressed(os.path.join(HERE, "fixpipe_qf322b8_values.npz"), data=data, quant_pre=q, golden=res)
    print("fixpipe_qf322b8_values", n)


QGMM = "examples/01_simd_cpp_api/05_best_practices/03_fusion_compute/quant_group_matmul_high_performance/scripts/gen_data.py"


def quant_group_matmul(reference, only=None):
    """The grouped W8A8 sample (G = 8, M = N = 8192, K = 1024, FastGelu, fp16 out): its generator runs unmodified with
    numpy's global seed fixed; the fixture keeps 16 rows of every group and the first 128 columns (an output element
    depends on its own row of x, its own column of its group's weight and the two scales only).  The weight file is
    written in the NZ layout [G, N/32, K/16, 16, 32]; it is brought back to [G, K, N] here."""
    path = os.path.join(reference, QGMM)
    G, M, K, N, rows_kept, cols_kept = 8, 8192, 1024, 8192, 16, 128
    with tempfile.TemporaryDirectory() as tmp:
        cwd = os.getcwd()
        os.chdir(tmp)
        try:
            np.random.seed(111)
            runpy.run_path(path, run_name="__main__")
            x = np.fromfile("input/x.bin", np.int8).reshape(M, K)
            w_nz = np.fromfile("input/weight.bin", np.int8).reshape(G, N // 32, K // 16, 16, 32)
            w = w_nz.transpose(0, 2, 3, 1, 4).reshape(G, K, N)
            groups = np.fromfile("input/groupList.bin", np.int64)
            scale = np.fromfile("input/scale.bin", np.float32).reshape(G, N)
            tok = np.fromfile("input/perTokenScale.bin", np.float32).reshape(M)
            golden = np.fromfile("output/golden.bin", np.float16).reshape(M, N)
        finally:
            os.chdir(cwd)
    starts = np.concatenate([[0], np.cumsum(groups)])
    rows = np.concatenate([np.arange(starts[g], starts[g] + rows_kept) for g in range(G)])
    out = {"x": np.ascontiguousarray(x[rows]), "weight_gkn": np.ascontiguousarray(w[:, :, :cols_kept]),
           "groupList": np.full(G, rows_kept, np.int64), "scale": np.ascontiguousarray(scale[:, :cols_kept]),
           "perTokenScale": np.ascontiguousarray(tok[rows]), "golden": np.ascontiguousarray(golden[rows][:, :cols_kept])}
    np.savez_compressed(os.path.join(HERE, "quant_group_matmul.npz"), **out)
    print("quant_group_matmul", {k: v.shape for k, v in out.items()})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("ASC_DEVKIT_ROOT"), help="root of the asc-devkit tree (or set ASC_DEVKIT_ROOT)")
    ap.add_argument("--only", default=None, help="regenerate one fixture only (its name)")
    args = ap.parse_args()
    if not args.reference:
        ap.error("give --reference /path/to/asc-devkit or set ASC_DEVKIT_ROOT")
    if args.only == "quant_group_matmul":
        quant_group_matmul(args.reference)
        return
    for name, script, argv, seed, files in CASES:
        if args.only and args.only != name:
            continue
        path = os.path.join(args.reference, script)
        with tempfile.TemporaryDirectory() as tmp:
            cwd, old_argv = os.getcwd(), sys.argv
            os.chdir(tmp)
            try:
                if seed is not None:
                    np.random.seed(seed)
                sys.argv = [path] + argv
                runpy.run_path(path, run_name="__main__")
                out = {}
                for rel, (dt, shape) in files.items():
                    key = os.path.splitext(os.path.basename(rel))[0]
                    out[key] = np.fromfile(os.path.join(tmp, rel), dtype=dt).reshape(shape)
            finally:
                os.chdir(cwd)
                sys.argv = old_argv
        if name.startswith("matmul_quant"):   # 96 of the 1024 rows of A and of the golden keep the fixture small
            out["x1_gm"] = out["x1_gm"][:KEEP_ROWS].copy()
            out["golden"] = out["golden"][:KEEP_ROWS].copy()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, {k: v.shape for k, v in out.items()})
    if args.only:
        return
    fixpipe_req8(args.reference)
    fixpipe_qf322b8(args.reference)
    quant_group_matmul(args.reference)


if __name__ == "__main__":
    main()
