#!/usr/bin/env python3
"""Runs device code of NKKdev/TFFinfer itself on small inputs and keeps what it computes
(tests/golden/reference_outputs.npz), so that the plain implementation of the tests
(tests/plain_qwen3.py) rests on outputs of the reference and not on a reading of it alone.

    TFF_REFERENCE_DIR=/path/to/TFFinfer python tests/golden/make_reference_golden.py --out DIR

Needs a CUDA device and nvcc.  The reference as a whole does not build offline (its CMake
fetches glog, Taskflow and libdivide), but these kernels depend on nothing of the project:
the script cuts them out of the reference's files AT RUN TIME -- everything between
``namespace tff::kernel {`` and the first host-side declaration of each file -- into a
header in a temporary folder and compiles it with the small driver below.  No line of the
reference is stored in this repository.  What is run, with the reference's own launch
geometry and template arguments:

  src/kernel/cuda/norm.cu                   rms_norm_kernel_cuda_impl<float, 32, 32>   (launch as :129-139)
  src/kernel/cuda/rope_table.cu             precompute_rope_table<float, 8, 1, 64, 32> (launch as :53-63)
  src/kernel/cuda/unary.cu                  op_unary<float, op_silu>                   (launch as :53-60)
  src/kernel/cuda/paged_flash_attention.cu  paged_flash_attention_fp16_8x32<half, int64_t, 1, 1, 32, 8, 128, 8, 32,
                                            8, 4, 2, 3, 4, 32, 256> (launch as :1078-1097): rotate-half rotation of
                                            q and k from the table, causal mask (values as src/kernel/cuda/mask_op.cu:39-45),
                                            softmax attention of 32 query heads on 8 key/value heads of 128

The attention cases keep the new-token count a multiple of 8 and the key count a multiple of
32: for other counts the reference's tile loaders zero-fill through ``swizzle`` offsets that
were computed for another layout, which is outside what these cases want to pin.
The inputs are those of tests/golden/golden_inputs.py; tests/test_reference_golden.py compares
the plain implementation with the kept outputs.
"""
from __future__ import annotations

import argparse
import os
import re
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import golden_inputs as gi  # noqa: E402

# file -> regular expression of the first line that is no longer device code
CUTS = {
    "src/kernel/cuda/norm.cu": r"^\s*static void rms_norm_kernel_cuda\(",
    "src/kernel/cuda/rope_table.cu": r"^\s*class PreRopeTable<",
    "src/kernel/cuda/unary.cu": r"^\s*class UnaryOP<",
    "src/kernel/cuda/paged_flash_attention.cu": r"^\s*void paged_flash_attention_128\(",
}


def excerpt(path: str, stop: str) -> str:
    """The file's text from ``namespace tff::kernel {`` up to the declaration that matches ``stop``
    (the ``template<...>`` header in front of it left out), and the namespace closed."""
    lines = open(path, encoding="utf-8", errors="replace").read().split("\n")
    first = next(i for i, l in enumerate(lines) if l.startswith("namespace tff::kernel"))
    defines = [l for l in lines[:first] if l.startswith("#define")]
    end = next(i for i, l in enumerate(lines) if i > first and re.search(stop, l))
    k = end - 1
    while not lines[k].lstrip().startswith("template"):     # walk back over the template header
        k -= 1
    return "\n".join(defines + lines[first:k] + ["}  // namespace tff::kernel", ""])


DRIVER = r"""
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cmath>
#include <string>
#include <vector>
#include <algorithm>
using std::max;
using std::min;
// Declared only: the interleaved-pair rotation helpers of the excerpt (not the rotate-half ones that are
// run here) name this function of src/kernel/include/kernel_util.h:62; they are never instantiated.
namespace tff::kernel { __device__ half2 complex_mul_half2(const half2 &a, const half2 &b); }
#include "reference_excerpts.cuh"

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
    fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_)); return 3; } } while (0)

template <typename T> static std::vector<T> read_file(const std::string &p, size_t n) {
    std::vector<T> v(n);
    FILE *f = fopen(p.c_str(), "rb");
    if (!f || fread(v.data(), sizeof(T), n, f) != n) { fprintf(stderr, "cannot read %s\n", p.c_str()); exit(2); }
    fclose(f);
    return v;
}
template <typename T> static void write_file(const std::string &p, const std::vector<T> &v) {
    FILE *f = fopen(p.c_str(), "wb");
    if (!f || fwrite(v.data(), sizeof(T), v.size(), f) != v.size()) { fprintf(stderr, "cannot write %s\n", p.c_str()); exit(2); }
    fclose(f);
}
template <typename T> static T *to_device(const std::vector<T> &v) {
    T *d = nullptr;
    if (cudaMalloc(&d, v.size() * sizeof(T)) != cudaSuccess) exit(3);
    cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice);
    return d;
}

int main(int argc, char **argv) {
    if (argc < 3) return 2;
    const std::string what = argv[1], dir = argv[2];
    using namespace tff::kernel;
    if (what == "norm") {            // norm DIR rows heads dim eps
        const int rows = atoi(argv[3]), heads = atoi(argv[4]), dim = atoi(argv[5]);
        const float eps = (float) atof(argv[6]);
        auto x = read_file<float>(dir + "/x.f32", (size_t) rows * heads * dim);
        auto w = read_file<float>(dir + "/w.f32", dim);
        float *dx = to_device(x), *dw = to_device(w), *dy = nullptr;
        CK(cudaMalloc(&dy, x.size() * 4));
        const dim3 grid(heads, (rows + 31) / 32, 1), block(32, 8, 1);
        rms_norm_kernel_cuda_impl<float, 32, 32><<<grid, block>>>(eps, dim, heads, rows, 1, dx, dw, dy);
        CK(cudaGetLastError());
        CK(cudaDeviceSynchronize());
        std::vector<float> y(x.size());
        CK(cudaMemcpy(y.data(), dy, y.size() * 4, cudaMemcpyDeviceToHost));
        write_file(dir + "/y.f32", y);
    } else if (what == "rope") {     // rope DIR max_pos dim theta
        const int max_pos = atoi(argv[3]), dim = atoi(argv[4]);
        const float base = (float) atof(argv[5]);
        float *dt = nullptr;
        CK(cudaMalloc(&dt, (size_t) max_pos * dim * 4));
        const dim3 grid((dim / 2 + 31) / 32, (max_pos + 63) / 64), block(256, 1);
        precompute_rope_table<float, 8, 1, 64, 32><<<grid, block>>>(max_pos, dim, std::log(base), dt);
        CK(cudaGetLastError());
        CK(cudaDeviceSynchronize());
        std::vector<float> t((size_t) max_pos * dim);
        CK(cudaMemcpy(t.data(), dt, t.size() * 4, cudaMemcpyDeviceToHost));
        write_file(dir + "/table.f32", t);
    } else if (what == "silu") {     // silu DIR n
        const int64_t n = atoll(argv[3]);
        auto g = read_file<float>(dir + "/gate.f32", n), u = read_file<float>(dir + "/up.f32", n);
        float *dg = to_device(g), *du = to_device(u), *dy = nullptr;
        CK(cudaMalloc(&dy, n * 4));
        op_unary<float, op_silu><<<(unsigned) ((n + 255) / 256), 256>>>(dg, du, dy, n, n, n);
        CK(cudaGetLastError());
        CK(cudaDeviceSynchronize());
        std::vector<float> y(n);
        CK(cudaMemcpy(y.data(), dy, n * 4, cudaMemcpyDeviceToHost));
        write_file(dir + "/y.f32", y);
    } else if (what == "attention") {    // attention DIR start new theta
        constexpr int NQ = 32, NKV = 8, D = 128;
        const int start = atoi(argv[3]), M = atoi(argv[4]), N = start + M;
        const float base = (float) atof(argv[5]);
        if (M % 8 || N % 32) { fprintf(stderr, "counts outside the cases this driver is for\n"); return 2; }
        auto q = read_file<__half>(dir + "/q.f16", (size_t) M * NQ * D);
        auto k = read_file<__half>(dir + "/k.f16", (size_t) N * NKV * D);
        auto v = read_file<__half>(dir + "/v.f16", (size_t) N * NKV * D);
        __half *dq = to_device(q), *dk = to_device(k), *dv = to_device(v);
        // one pointer per (token, key/value head), as the reference's cache hands keys and values to the kernel
        std::vector<int64_t> kp((size_t) N * NKV), vp((size_t) N * NKV);
        for (int t = 0; t < N; ++t)
            for (int h = 0; h < NKV; ++h) {
                kp[(size_t) t * NKV + h] = (int64_t) (dk + ((size_t) t * NKV + h) * D);
                vp[(size_t) t * NKV + h] = (int64_t) (dv + ((size_t) t * NKV + h) * D);
            }
        int64_t *dkp = to_device(kp), *dvp = to_device(vp);
        // mask[query position][key position]: 0 where the key is not after the query, -inf elsewhere
        std::vector<__half> mask((size_t) N * N);
        for (int r = 0; r < N; ++r)
            for (int c = 0; c < N; ++c) mask[(size_t) r * N + c] = __float2half(r >= c ? 0.0f : -INFINITY);
        __half *dmask = to_device(mask);
        float *dt = nullptr, *dout = nullptr;
        CK(cudaMalloc(&dt, (size_t) N * D * 4));
        const dim3 tgrid((D / 2 + 31) / 32, (N + 63) / 64), tblock(256, 1);
        precompute_rope_table<float, 8, 1, 64, 32><<<tgrid, tblock>>>(N, D, std::log(base), dt);
        CK(cudaGetLastError());
        CK(cudaMalloc(&dout, (size_t) M * NQ * D * 4));
        CK(cudaMemset(dout, 0, (size_t) M * NQ * D * 4));
        const dim3 grid((M + 7) / 8, NQ / 4, 1), block(256);
        paged_flash_attention_fp16_8x32<__half, int64_t, 1, 1, NQ, NKV, D, 8, 32, 8, 4, 2, 3, 4, 32, 256>
            <<<grid, block>>>(start, N, M, N, D, D, 1, 1, 1.0f / std::sqrt((float) D), dq, dkp, dvp, dmask, dt, dout);
        CK(cudaGetLastError());
        CK(cudaDeviceSynchronize());
        std::vector<float> out((size_t) M * NQ * D);
        CK(cudaMemcpy(out.data(), dout, out.size() * 4, cudaMemcpyDeviceToHost));
        write_file(dir + "/out.f32", out);
    } else {
        return 2;
    }
    return 0;
}
"""


def run(exe, what, work, *args):
    cmd = [exe, what, work] + [repr(a) if isinstance(a, float) else str(a) for a in args]
    subprocess.run(cmd, check=True)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", default=HERE, help="folder reference_outputs.npz is written to")
    ap.add_argument("--arch", default="-gencode arch=compute_100a,code=sm_100a")
    args = ap.parse_args()
    ref = os.environ.get("TFF_REFERENCE_DIR")
    if not ref or not os.path.isdir(ref):
        print("set TFF_REFERENCE_DIR to a checkout of NKKdev/TFFinfer", file=sys.stderr)
        return 2
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        with open(os.path.join(tmp, "reference_excerpts.cuh"), "w") as f:
            for rel, stop in CUTS.items():
                f.write(f"// ---- cut at run time out of {rel}\n")
                f.write(excerpt(os.path.join(ref, rel), stop))
        with open(os.path.join(tmp, "driver.cu"), "w") as f:
            f.write(DRIVER)
        exe = os.path.join(tmp, "driver")
        subprocess.run(["nvcc", "-std=c++17", "-O2", *args.arch.split(), "-o", exe, os.path.join(tmp, "driver.cu")],
                       check=True)
        work = os.path.join(tmp, "work")
        os.makedirs(work)
        for name, c in gi.NORM_CASES.items():
            x, w = gi.norm_inputs(c)
            x.tofile(os.path.join(work, "x.f32"))
            w.tofile(os.path.join(work, "w.f32"))
            run(exe, "norm", work, c["rows"], c["heads"], c["dim"], c["eps"])
            out[name] = np.fromfile(os.path.join(work, "y.f32"), dtype=np.float32).reshape(x.shape)
        for name, c in gi.ROPE_CASES.items():
            run(exe, "rope", work, c["max_pos"], c["dim"], c["theta"])
            t = np.fromfile(os.path.join(work, "table.f32"), dtype=np.float32).reshape(c["max_pos"], c["dim"] // 2, 2)
            out[name] = t[c["keep"]].copy()
        c = gi.SILU_CASE
        gate, up = gi.silu_inputs(c)
        gate.tofile(os.path.join(work, "gate.f32"))
        up.tofile(os.path.join(work, "up.f32"))
        run(exe, "silu", work, c["n"])
        out["silu_mul"] = np.fromfile(os.path.join(work, "y.f32"), dtype=np.float32)
        g = gi.ATTENTION_GEOMETRY
        for name, c in gi.ATTENTION_CASES.items():
            q, k, v = gi.attention_inputs(c)
            q.tofile(os.path.join(work, "q.f16"))
            k.tofile(os.path.join(work, "k.f16"))
            v.tofile(os.path.join(work, "v.f16"))
            run(exe, "attention", work, c["start"], c["new"], g["theta"])
            o = np.fromfile(os.path.join(work, "out.f32"), dtype=np.float32).reshape(c["new"], g["heads"], g["head_dim"])
            kept = o[c["keep_rows"]]
            assert np.array_equal(kept.astype(np.float16).astype(np.float32), kept), \
                "the kernel's outputs are half-precision values widened; float16 storage must be exact"
            out[name] = kept.astype(np.float16)
    os.makedirs(args.out, exist_ok=True)
    path = os.path.join(args.out, "reference_outputs.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: " + ", ".join(f"{k}{list(v.shape)}" for k, v in out.items()))
    return 0


if __name__ == "__main__":
    sys.exit(main())
