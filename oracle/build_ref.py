#!/usr/bin/env python3
"""Build oracle/_ref/ from the Checkers reference sources where they lie.

TEST INFRASTRUCTURE ONLY.  Nothing here is shipped and no reference source is
copied into this repository: the function bodies named below are cut out of the
reference tree into a temporary directory, compiled together with
oracle/ref_shim.cpp (which supplies a CPU stand-in for threadIdx/__shared__/
__syncthreads and stub owner classes), and only the resulting binaries land in
oracle/_ref/:

  oracle/_ref/libcheckers_ref.so              reference kernel bodies, table
                                              normaliser, file writers, clustering
  oracle/_ref/tensor_group_prefix_mask_repair the reference Re-Pair CLI, unmodified

The reference's own build (CMake + RAJA + Umpire, GPU only) cannot run here, so
its orchestration code (thread pool, streams, allocators) is not part of this
build; the restatement in checkers_oracle.cpp covers it.

Usage: python oracle/build_ref.py [--reference /path/to/Checkers]
"""
import argparse
import os
import re
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))


def cut_block(text, start_regex, what):
    """Return the source text from the line matching start_regex through the
    brace that closes the first '{' after it (plus a trailing ';' if present)."""
    m = re.search(start_regex, text, re.M)
    if not m:
        raise SystemExit(f"build_ref: cannot find {what}")
    i = text.index("{", m.start())
    depth, j, n = 0, i, len(text)
    while j < n:
        c = text[j]
        if text.startswith("//", j):
            j = text.index("\n", j)
            continue
        if text.startswith("/*", j):
            j = text.index("*/", j) + 2
            continue
        if c == '"':
            j += 1
            while text[j] != '"':
                j += 2 if text[j] == "\\" else 1
        elif c == "'":
            j += 1
            while text[j] != "'":
                j += 2 if text[j] == "\\" else 1
        elif c == "{":
            depth += 1
        elif c == "}":
            depth -= 1
            if depth == 0:
                j += 1
                break
        j += 1
    if j < n and text[j] == ";":
        j += 1
    return text[m.start():j] + "\n"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CHECKERS_REFERENCE", ""),
                    help="the Checkers source tree (or set CHECKERS_REFERENCE)")
    args = ap.parse_args()
    ref = args.reference
    if not os.path.isdir(os.path.join(ref, "src")):
        print(f"build_ref: no reference tree at {ref}; skipping", file=sys.stderr)
        return 0
    out_dir = os.path.join(HERE, "_ref")
    os.makedirs(out_dir, exist_ok=True)

    rd = lambda p: open(os.path.join(ref, p)).read()
    ans_cpp = rd("src/ANSCompressor.cpp")
    ans_hpp = rd("include/checkers/ANSCompressor.hpp")
    ta_cpp = rd("src/TensorAnalyzer.cpp")
    tr_hpp = rd("include/checkers/TensorResource.hpp")
    mm_hpp = rd("include/checkers/MemoryManager.hpp")

    pieces = {
        # types and constants
        "types.inc": "".join([
            cut_block(tr_hpp, r"^enum class DataType\b", "DataType"),
            cut_block(tr_hpp, r"^struct TensorStatistics\b", "TensorStatistics"),
            cut_block(tr_hpp, r"^struct TensorFingerprint\b", "TensorFingerprint"),
            cut_block(mm_hpp, r"^struct DeviceTensorRecord\b", "DeviceTensorRecord"),
            cut_block(mm_hpp, r"^struct ClusterInfo\b", "ClusterInfo"),
            "".join(re.findall(r"^static constexpr uint32_t ANS_\w+\s*=.*$\n", ans_hpp, re.M)),
            cut_block(ans_hpp, r"^struct alignas\(64\) ANSFreqTable\b", "ANSFreqTable"),
            cut_block(ans_hpp, r"^struct ANSStreamHeader\b", "ANSStreamHeader"),
            cut_block(ans_hpp, r"^struct CompressedTensor\b", "CompressedTensor"),
        ]),
        "member_types.inc": "".join([
            cut_block(ans_hpp, r"^    struct SidecarInfo\b", "SidecarInfo"),
            cut_block(ans_hpp, r"^    struct SidecarEntry\b", "SidecarEntry"),
            cut_block(ans_hpp, r"^    struct TableEntry\b", "TableEntry"),
        ]),
        "kernels.inc": "".join([
            cut_block(ans_cpp, r"^__global__ void byte_histogram_kernel\b", "byte_histogram_kernel"),
            cut_block(ans_cpp, r"^__global__ void rans_encode_kernel\b", "rans_encode_kernel"),
            cut_block(ans_cpp, r"^__global__ void compact_streams_kernel\b", "compact_streams_kernel"),
            cut_block(ans_cpp, r"^__global__ void extract_mantissa_kernel\b", "extract_mantissa_kernel"),
        ]),
        "stats.inc": "".join([
            cut_block(ta_cpp, r"^template <typename T>\n__device__ void compute_tensor_stats\b", "compute_tensor_stats"),
            cut_block(ta_cpp, r"^__global__ void tensor_stats_kernel\b", "tensor_stats_kernel"),
        ]),
        "host.inc": "".join([
            "".join(re.findall(r"^static constexpr uint32_t (?:ANSC|DICT|MANT)_\w+\s*=.*$\n", ans_cpp, re.M)),
            cut_block(ans_cpp, r"^ANSFreqTable ANSCompressor::normalize_histogram\b", "normalize_histogram"),
            cut_block(ans_cpp, r"^void ANSCompressor::write_rank_states_file\b", "write_rank_states_file"),
            cut_block(ans_cpp, r"^void ANSCompressor::write_rank_mantissa_file\b", "write_rank_mantissa_file"),
            cut_block(ans_cpp, r"^void ANSCompressor::write_rank_tables_file\b", "write_rank_tables_file"),
        ]),
        "cluster.inc": cut_block(ta_cpp, r"^void TensorAnalyzer::build_knn_clusters\b", "build_knn_clusters"),
    }

    with tempfile.TemporaryDirectory(prefix="chk_ref_") as tmp:
        for name, src in pieces.items():
            with open(os.path.join(tmp, name), "w") as f:
                f.write(src)
        so = os.path.join(out_dir, "libcheckers_ref.so")
        cmd = ["g++", "-std=c++20", "-O2", "-ffp-contract=off", "-fno-stack-protector", "-fPIC", "-shared",
               "-w", "-I", tmp, os.path.join(HERE, "ref_shim.cpp"), "-o", so]
        subprocess.check_call(cmd)
        print("built", so)

    cli = os.path.join(out_dir, "tensor_group_prefix_mask_repair")
    subprocess.check_call(["g++", "-std=c++20", "-O2", "-w",
                           os.path.join(ref, "src/tensor_group_prefix_mask_repair.cpp"), "-o", cli])
    print("built", cli)
    return 0


if __name__ == "__main__":
    sys.exit(main())
