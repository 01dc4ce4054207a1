"""The GEMV's in-place code decode (lisa_b200/csrc/qmv_math.h) compiled for the host:
t = 1 + q * 2^(P-23) and t * (x * 2^(23-P)) - x * 2^(23-P) == q * x for every code position."""
import os
import subprocess
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SRC = r"""
#include <cstdio>
#include <cstring>
#include <cstdint>
#include <cmath>
#include "qmv_math.h"
using namespace lisa;
static float as_f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
template <int BITS> int run() {
    using C = QmvCode<BITS>;
    uint32_t state = 12345u;
    int bad = 0;
    for (int it = 0; it < 20000; ++it) {
        state = state * 1664525u + 1013904223u;
        uint32_t w = state ^ (state << 7);
        uint32_t lo[C::kPairsPerWord], hi[C::kPairsPerWord];
        C::decode(w, lo, hi);
        int seen[C::kCodesPerWord] = {0};
        for (int p = 0; p < C::kPairsPerWord; ++p)
            for (int e = 0; e < 2; ++e) {
                int j = C::code_of(p, e);
                seen[j]++;
                uint32_t q = (w >> (j * BITS)) & ((1u << BITS) - 1u);
                float t = as_f(e == 0 ? lo[p] : hi[p]);
                float xs = C::xscale_of(p, e);  // x = 1
                float got = t * xs - xs;        // exact: t has few bits
                if (got != (float)q) { if (bad < 5) printf("bits %d w %08x p %d e %d j %d got %g want %u\n", BITS, w, p, e, j, got, q); bad++; }
            }
        for (int j = 0; j < C::kCodesPerWord; ++j) if (seen[j] != 1) { bad++; }
    }
    return bad;
}
int main() { int b = run<4>() + run<2>(); printf("bad=%d\n", b); return b != 0; }
"""


def test_decode_positions_and_scales():
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "t.cc")
        exe = os.path.join(tmp, "t")
        open(src, "w").write(SRC)
        subprocess.run(["g++", "-O1", "-std=c++17", "-I", os.path.join(ROOT, "lisa_b200", "csrc"), src, "-o", exe],
                       check=True)
        res = subprocess.run([exe], capture_output=True, text=True)
        assert res.returncode == 0, res.stdout
        assert "bad=0" in res.stdout
