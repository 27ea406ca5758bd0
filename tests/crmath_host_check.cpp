// TEST INFRASTRUCTURE.  Compiles repdl_b200/csrc/crmath.cuh for the HOST and compares cr_exp /
// cr_log with glibc's (float)exp((double)x) / (float)log((double)x) -- the reference's definition
// (microsoft/RepDL backend/cpu/math.cpp:14-17, 32-35) -- over a strided sweep of ALL fp32 bit
// patterns.  stride 1 is the exhaustive run (2^32 inputs per function).
//
// The `div` mode checks the scalar division of the streaming kernel (cr_div_by_reciprocal with its
// exact fall-back) against the IEEE quotient x / d (microsoft/RepDL repdl/ops.py:98-103).
//
//   g++ -O2 -ffp-contract=off -mfma -fopenmp [-DCRM_FORCE_SLOW=1] tests/crmath_host_check.cpp -o chk
//   ./chk exp|log <stride> <offset>       prints "<checked> <mismatches>"
//   ./chk div <stride> <offset> <d>       the same for x / d
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "../repdl_b200/csrc/crmath.cuh"

using namespace repdl_b200;

int main(int argc, char **argv)
{
    if (argc < 4) return 2;
    const bool is_exp = std::strcmp(argv[1], "exp") == 0;
    const bool is_div = std::strcmp(argv[1], "div") == 0;
    const float dv = is_div && argc > 4 ? std::strtof(argv[4], 0) : 1.0f;
    const double rd = 1.0 / (double)dv;
    const uint64_t stride = std::strtoull(argv[2], 0, 10), offset = std::strtoull(argv[3], 0, 10);
    uint64_t checked = 0, bad = 0;
#pragma omp parallel for schedule(dynamic, 1) reduction(+ : checked, bad)
    for (uint64_t blk = 0; blk < 4096; blk++) {
        const uint64_t lo = blk << 20, hi = lo + (1ull << 20);
        uint64_t first = lo + ((offset + stride - lo % stride) % stride);
        for (uint64_t u = first; u < hi; u += stride) {
            float x = crm_from_fbits((uint32_t)u);
            float want, got;
            if (is_div) {
                bool slow;
                want = x / dv;
                got = cr_div_by_reciprocal(x, rd, slow);
                if (slow) got = cr_div(x, dv);
                if (want != want && got != got) want = got;  // NaN payloads: checked by the special-value cases
            } else {
                want = is_exp ? (float)std::exp((double)x) : (float)std::log((double)x);
                got = is_exp ? cr_exp(x) : cr_log(x);
            }
            checked++;
            if (crm_fbits(want) != crm_fbits(got)) {
                bad++;
#pragma omp critical
                if (bad < 20)
                    std::printf("MISMATCH x=0x%08x want=0x%08x got=0x%08x\n", (unsigned)u,
                                crm_fbits(want), crm_fbits(got));
            }
        }
    }
    std::printf("%llu %llu\n", (unsigned long long)checked, (unsigned long long)bad);
    return bad ? 1 : 0;
}
