#!/usr/bin/env python3
"""Builds the reference arm: the UNMODIFIED sources of zscey/tiny-llm plus baseline/ref_driver.cpp.

    python baseline/build_reference.py [--reference /path/to/tiny-llm] [--jobs N]

pip cannot install the reference (it is a Bazel + Rust project without setup.py or pyproject.toml), but
its engine below the tokenizer is plain C++20 and CUDA.  This script copies its `tiny_llm/` tree, byte for
byte, into baseline/_ref/src/ (a folder outside the history), compiles the parts the engine needs with
nvcc for sm_100 and links them with the driver into baseline/_ref/ref_driver.  Left out, because they are
Rust behind a C interface or Bazel glue: tokenizers/, weight_managers/safetensors/, utils/runfile.cpp;
ops/cpu and thread_pool serve only the temperature processor, which the greedy driver does not use.

Headers the reference expects and this image carries inside Python packages (found at run time, nothing
is copied): spdlog with its bundled fmt, nlohmann/json, and a CCCL that has <cuda/warp> (the reference
targets CUDA 13 and includes it as "cccl/cuda/warp"; CUDA 12.9's own CCCL is older).  The include names
"cccl/..." and "fmt/..." are given to the compiler through two symlinks under baseline/_ref/shim/.
"""
import argparse
import concurrent.futures
import os
import shutil
import site
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SOURCES = [
    "tiny_llm/tensor/tensor.cpp",
    "tiny_llm/device_managers/buffer.cpp", "tiny_llm/device_managers/copy_data.cpp",
    "tiny_llm/device_managers/cpu/cpu_allocator.cpp",
    "tiny_llm/device_managers/cuda/cuda_allocator.cpp", "tiny_llm/device_managers/cuda/cuda_context.cpp",
    "tiny_llm/device_managers/cuda/cuda_device_guard.cpp", "tiny_llm/device_managers/cuda/cuda_device_infos.cpp",
    "tiny_llm/graph/graph.cpp", "tiny_llm/graph/param.cpp",
    "tiny_llm/parser/llama_parser.cpp",
    "tiny_llm/runtime/page_pool.cpp", "tiny_llm/runtime/greedy_memory_planer.cpp",
    "tiny_llm/runtime/cuda/cuda_kernels.cpp", "tiny_llm/runtime/cuda/cuda_plan.cpp", "tiny_llm/runtime/cuda/cuda_runtime.cpp",
    "tiny_llm/logit_processors/argmax_processor.cpp",
    "tiny_llm/ops/cuda/arithmetic.cu", "tiny_llm/ops/cuda/embedding.cu", "tiny_llm/ops/cuda/flash_attention.cu",
    "tiny_llm/ops/cuda/gemm.cu", "tiny_llm/ops/cuda/gemm_q1_helper.cu", "tiny_llm/ops/cuda/norm.cu",
    "tiny_llm/ops/cuda/rope.cu", "tiny_llm/ops/cuda/silu.cu",
]


def find_headers():
    """Include folders for spdlog (+ bundled fmt), nlohmann/json and a CCCL with <cuda/warp>."""
    roots = list(site.getsitepackages()) + [site.getusersitepackages()]
    found = {}
    for r in roots:
        for key, rel in (("spdlog", "flashinfer/data/spdlog/include"), ("cccl", "flashinfer/data/cccl"),
                         ("json", "include/cudnn_frontend/thirdparty")):
            p = os.path.join(r, rel)
            if key not in found and os.path.isdir(p):
                found[key] = p
    missing = [k for k in ("spdlog", "cccl", "json") if k not in found]
    if missing:
        raise SystemExit(f"build_reference: headers not found in the Python packages of this image: {missing}")
    return found


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("TLLM_REFERENCE", os.path.join(HERE, "..", "..", "reference")),
                    help="a tiny-llm checkout (default: TLLM_REFERENCE, else the folder `reference` beside this repository)")
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    ap.add_argument("--arch", default="sm_100")
    args = ap.parse_args()
    src = os.path.join(OUT, "src")
    if os.path.isdir(os.path.join(args.reference, "tiny_llm")):
        if os.path.isdir(src):
            shutil.rmtree(src)
        os.makedirs(src)
        shutil.copytree(os.path.join(args.reference, "tiny_llm"), os.path.join(src, "tiny_llm"))
    elif not os.path.isdir(os.path.join(src, "tiny_llm")):
        raise SystemExit(f"build_reference: no reference checkout at {args.reference} and no copy under {src}")
    h = find_headers()
    shim = os.path.join(OUT, "shim")
    os.makedirs(shim, exist_ok=True)
    for name, target in (("cccl", os.path.join(h["cccl"], "libcudacxx", "include")),
                         ("fmt", os.path.join(h["spdlog"], "spdlog", "fmt", "bundled"))):
        link = os.path.join(shim, name)
        if os.path.islink(link):
            os.remove(link)
        os.symlink(target, link)
    inc = ["-I", src, "-I", shim, "-I", os.path.join(h["cccl"], "libcudacxx", "include"), "-I", os.path.join(h["cccl"], "cub"),
           "-I", os.path.join(h["cccl"], "thrust"), "-I", h["spdlog"], "-I", h["json"], "-DFMT_HEADER_ONLY",
           # what the reference's BUILD files define on a CUDA platform (tiny_llm/device_managers/BUILD:18-19,
           # tiny_llm/tensor/BUILD:9-10)
           "-DTINY_LLM_COPY_DATA_WITH_CUDA", "-DTINY_LLM_TENSOR_WITH_CUDA"]
    flags = ["-std=c++20", "-O3", f"-arch={args.arch}", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-w"]
    obj_dir = os.path.join(OUT, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"

    def compile_one(rel_or_abs):
        path = rel_or_abs if os.path.isabs(rel_or_abs) else os.path.join(src, rel_or_abs)
        obj = os.path.join(obj_dir, os.path.basename(path).rsplit(".", 1)[0] + ".o")
        cmd = [nvcc] + flags + inc + ["-x", "cu", "-c", path, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        return path, obj, res

    objs, failed = [], []
    with concurrent.futures.ThreadPoolExecutor(max_workers=args.jobs) as pool:
        for path, obj, res in pool.map(compile_one, SOURCES + [os.path.join(HERE, "ref_driver.cpp")]):
            print(("ok    " if res.returncode == 0 else "FAILED") + " " + os.path.relpath(path, OUT), flush=True)
            if res.returncode != 0:
                failed.append((path, res.stdout + res.stderr))
            objs.append(obj)
    if failed:
        with open(os.path.join(OUT, "build_errors.log"), "w") as f:
            for path, log in failed:
                f.write(f"==== {path}\n{log}\n")
        print(failed[0][1][-3000:], file=sys.stderr)
        raise SystemExit(f"build_reference: {len(failed)} file(s) did not compile; see baseline/_ref/build_errors.log")
    exe = os.path.join(OUT, "ref_driver")
    res = subprocess.run([nvcc, f"-arch={args.arch}", "-o", exe] + objs + ["-lcudart"], capture_output=True, text=True)
    if res.returncode != 0:
        print(res.stdout + res.stderr, file=sys.stderr)
        raise SystemExit("build_reference: link failed")
    print("built", os.path.relpath(exe, os.path.dirname(HERE)))


if __name__ == "__main__":
    main()
