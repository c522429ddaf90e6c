#!/usr/bin/env python3
"""Makes tests/golden/reference_ops.json from the reference's own CPU oracles.

wiketool/ToyInfer's model code is CUDA only and cannot run without a GPU, but the CPU
reference functions of its kernel tests (tests/*_test_common.h) compile with g++.  This
script writes a small driver (below, ours) that includes those headers from a checkout of
the reference, builds the reference's own test inputs with its ``make_case`` functions,
rounds them to bfloat16 as its tests do, calls its ``reference_output`` functions, and
dumps inputs and outputs as JSON.  tests/test_golden.py feeds the same inputs to the plain
implementation and compares.

    python tests/golden/make_golden.py /path/to/ToyInfer [/usr/local/cuda/include]

The committed JSON was made this way; the whole-model composition has no such anchor.
"""
import os
import subprocess
import sys
import tempfile

DRIVER = r'''
#include <cstdio>
#include <vector>
#include "test_helpers.h"
#include "rmsnorm_test_common.h"
#include "multi_rmsnorm_test_common.h"
#include "rope_test_common.h"
#include "swiglu_test_common.h"
#include "flash_attention_test_common.h"
#include "precompute_freq_test_common.h"
#include "gemv_test_common.h"
#include "attention_test_common.h"
#include "add_test_common.h"

static std::vector<float> q(const std::vector<float>& v) { return kernel_test::to_float(kernel_test::to_bf16(v)); }
static void dump(const char* name, const std::vector<float>& v, size_t n, bool last = false) {
    printf("  \"%s\": [", name);
    for (size_t i = 0; i < n; i++) printf("%s%.9g", i ? "," : "", v[i]);
    printf("]%s\n", last ? "" : ",");
}
int main() {
    printf("{\n");
    {   // RMS norm over 258 elements (src/decode.cu:99-125)
        auto c = rmsnorm_test::make_case("g", 258, 258, 1e-5f, 0.37f, 0.21f);
        auto x = q(c.input), w = q(c.weight);
        std::vector<float> init(258, 0.f);
        auto y = rmsnorm_test::reference_output(x, w, init, rmsnorm_test::reference_sum(x, 258), c.eps, 258);
        printf(" \"rmsnorm\": {\n  \"eps\": 1e-5,\n"); dump("x", x, 258); dump("w", w, 258); dump("y", y, 258, true); printf(" },\n");
    }
    {   // per-head RMS norm, 3 heads of 32 (src/decode.cu:144-187)
        auto c = multi_rmsnorm_test::make_case("g", 3, 32, 96, 1e-6f, false, 0.29f, 0.17f);
        auto x = q(c.input), w = q(c.weight);
        std::vector<float> init(96, 0.f);
        auto y = multi_rmsnorm_test::reference_output(c, x, w, init);
        printf(" \"head_rmsnorm\": {\n  \"eps\": 1e-6, \"heads\": 3, \"head_dim\": 32,\n"); dump("x", x, 96); dump("w", w, 32); dump("y", y, 96, true); printf(" },\n");
    }
    {   // rotation, 2 heads of 16 at position 7 (src/decode.cu:301-324)
        auto c = rope_test::make_case("g", 2, 16, 7, 32, 0.41f, 0.013f);
        auto x = q(c.qk);
        auto y = rope_test::reference_output(c, x);
        printf(" \"rope\": {\n  \"heads\": 2, \"head_dim\": 16, \"pos\": 7,\n"); dump("x", x, 32); dump("inv_freq", c.inv_freq, 8); dump("y", y, 32, true); printf(" },\n");
    }
    {   // SwiGLU over 200 elements (src/decode.cu:746-764)
        auto c = swiglu_test::make_case("g", 200, 200, 0.23f, 0.31f);
        auto g = q(c.gate), u = q(c.up);
        std::vector<float> init(200, 0.f);
        auto y = swiglu_test::reference_output(g, u, init, 200);
        printf(" \"swiglu\": {\n"); dump("gate", g, 200); dump("up", u, 200); dump("y", y, 200, true); printf(" },\n");
    }
    {   // causal grouped-query attention: 4 heads over 2 kv heads of 16, 9 positions (src/prefill.cu:224-379)
        auto c = flash_attention_test::make_case("g", 4, 2, 16, 9, 0.19f, 0.23f);
        auto qq = q(c.q), k = q(c.ks), v = q(c.vs);
        auto y = flash_attention_test::reference_output(c, qq, k, v);
        printf(" \"attention\": {\n  \"heads\": 4, \"kv_heads\": 2, \"head_dim\": 16, \"seq\": 9,\n");
        dump("q", qq, qq.size()); dump("k", k, k.size()); dump("v", v, v.size()); dump("y", y, y.size(), true); printf(" },\n");
    }
    {   // rotation frequencies (src/decode.cu:35-41)
        precompute_freq_test::Case c; c.head_dim = 32; c.buffer_size = 16; c.theta = 1000000.0f;
        std::vector<float> init(16, 0.f);
        auto y = precompute_freq_test::build_expected(c, init);
        printf(" \"inv_freq\": {\n  \"head_dim\": 32, \"theta\": 1000000.0,\n"); dump("y", y, 16, true); printf(" },\n");
    }
    {   // matrix times vector, 5 rows of 12: weights [out, in] row-major (src/decode.cu:202-236)
        auto c = gemv_test::make_case("g", 5, 12, 5, 0.31f, 0.17f);
        auto x = q(c.x), w = q(c.w);
        auto y = gemv_test::reference_sum(c, x, w);
        printf(" \"gemv\": {\n  \"rows\": 5, \"cols\": 12,\n"); dump("x", x, 12); dump("w", w, 60); dump("y", y, 5, true); printf(" },\n");
    }
    {   // one token's attention over cache rows 0..pos: scores, softmax, weighted values
        // (src/decode.cu:401-432, :471-532, :598-628); 6 heads over 2 kv heads of 8, position 10 of 16 rows
        auto c = attention_test::make_attention_case("g", 6, 2, 8, 10, 16, 0.27f, 0.19f);
        auto qq = q(c.q), k = q(c.ks), v = q(c.vs);
        std::vector<float> zeros(6 * 16, 0.f);
        auto scores = attention_test::reference_qk_scores(c, qq, k, zeros);
        auto probs = attention_test::reference_attention_score(c, qq, k);
        auto o = attention_test::reference_attention_buffer(c, probs, v);
        printf(" \"decode_attention\": {\n  \"heads\": 6, \"kv_heads\": 2, \"head_dim\": 8, \"pos\": 10, \"rows\": 16,\n");
        dump("q", qq, qq.size()); dump("k", k, k.size()); dump("v", v, v.size()); dump("scores", scores, scores.size());
        dump("probs", probs, probs.size()); dump("o", o, o.size(), true); printf(" },\n");
    }
    {   // residual sum, rounded to bfloat16 (src/decode.cu:7-22)
        auto c = add_test::make_case("g", 50, 50, false, 0.21f, 0.33f, 0.0f);
        auto r = q(c.residual), h = q(c.hidden);
        auto y = add_test::apply_reference(h, r, 50);
        printf(" \"residual_add\": {\n"); dump("residual", r, 50); dump("hidden", h, 50); dump("y", y, 50, true); printf(" }\n");
    }
    printf("}\n");
    return 0;
}
'''


def main() -> int:
    if len(sys.argv) < 2:
        print(__doc__)
        return 2
    ref = sys.argv[1]
    cuda_inc = sys.argv[2] if len(sys.argv) > 2 else "/usr/local/cuda/include"
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_ops.json")
    with tempfile.TemporaryDirectory() as d:
        src, exe = os.path.join(d, "driver.cpp"), os.path.join(d, "driver")
        with open(src, "w") as f:
            f.write(DRIVER)
        subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ref, "tests"), "-I", cuda_inc, src, "-o", exe],
                       check=True)
        text = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
    with open(out, "w") as f:
        f.write(text)
    print("wrote", out, len(text), "bytes")
    return 0


if __name__ == "__main__":
    sys.exit(main())
