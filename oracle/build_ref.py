"""Compile the reference's own CUDA kernels for sm_100a into oracle/_ref/.

TEST INFRASTRUCTURE ONLY.  The reference keeps its kernels as CUDA-C string
constants inside Rust sources.  This script reads those constants from the
reference tree where it lies, writes them unchanged into a scratch directory,
and compiles them together with ``ref_launch.cu`` (host launchers written for
this repository) into ``oracle/_ref/libtwm_ref.so``.  Only that binary is kept;
no reference source enters the repository.

Usage:  python oracle/build_ref.py [--reference /path/to/reference]
Without a reference tree the script reports that and exits 0: the machine
that runs the GPU tests uses the prebuilt library.
"""
from __future__ import annotations

import argparse
import os
import re
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT_SO = os.path.join(OUT_DIR, "libtwm_ref.so")

# (file under crates/kernels/src, constant name): the kernel string it holds
WANTED = [
    ("quantize.rs", "QUANTIZE_Q4_0_SRC"),                       # quantize.rs:103-146
    ("quantize.rs", "DEQUANTIZE_Q4_0_SRC"),                     # quantize.rs:150-175
    ("quantize.rs", "GEMM_Q4_0_SRC"),                           # quantize.rs:186-246
    ("quantize.rs", "DEQUANT_Q4_TO_F16_SRC"),                   # quantize.rs:534-571
    ("quantize.rs", "GEMM_TW_MARLIN_M1_SRC"),                   # quantize.rs:1186-1245
    ("quantize.rs", "GEMM_TW_MARLIN_M1_DIRECT_SRC"),            # quantize.rs:1249-1298
    ("moe_batched_marlin.rs", "BATCHED_MARLIN_GATE_UP_SRC"),    # moe_batched_marlin.rs:21-74
    ("moe_batched_marlin.rs", "BATCHED_MARLIN_DOWN_AXPY_SRC"),  # moe_batched_marlin.rs:78-134
    ("moe_batched_marlin.rs", "BATCHED_SPLIT_GEGLU_SRC"),       # moe_batched_marlin.rs:138-152
]


def extract(rs_text: str, name: str) -> str:
    m = re.search(r"const\s+" + re.escape(name) + r'\s*:\s*&str\s*=\s*r#"(.*?)"#;', rs_text, re.S)
    if not m:
        raise RuntimeError(f"kernel constant {name} not found in the reference source")
    return m.group(1)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("TWM_REFERENCE_ROOT", "/root/reference"))
    args = ap.parse_args()
    src_dir = os.path.join(args.reference, "crates", "kernels", "src")
    if not os.path.exists(os.path.join(src_dir, "quantize.rs")):
        print(f"build_ref: no reference tree at {args.reference}; keeping any prebuilt {OUT_SO}")
        return 0
    texts = {}
    for fname in sorted({f for f, _ in WANTED}):
        with open(os.path.join(src_dir, fname), "r", encoding="utf-8") as f:
            texts[fname] = f.read()
    os.makedirs(OUT_DIR, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        inc = os.path.join(tmp, "ref_kernels.inc")
        with open(inc, "w", encoding="utf-8") as f:
            for fname, name in WANTED:
                body = extract(texts[fname], name)
                # two constants define the same helper macro name TILE; keep each body self-contained
                f.write(f"// ---- {name}\n{body}\n#undef TILE\n")
        cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-shared",
               "-Xcompiler", "-fPIC", f"-DREF_KERNELS_INC=\"{inc}\"",
               os.path.join(HERE, "ref_launch.cu"), "-o", OUT_SO]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            return r.returncode
    print(f"build_ref: wrote {OUT_SO}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
