// The arithmetic of the summarised fp32 chain sum (sum1d.cu), written once for the device and for
// the host: the CUDA kernels include this header, and so does the host model of the pipeline that
// the CPU test-suite compiles with g++ and checks against the plain chain (tests/sum1d_host_model.cpp).
//
// Why a chain can be summarised.  While the running sum s stays inside one binade (exponent field
// E, ulp u = 2^(E-150)), s = m*u with an integer 2^23 <= |m| < 2^24, and a rounded fp32 add of
// x = q*u gives exactly m' = m + rint(q), rint = round-half-even; on an exact tie (q = n + 1/2) the
// result is whichever of m+n, m+n+1 is even, i.e. it depends on the parity of m.  So, for a fixed
// binade hypothesis E, a run of elements acts on m as  m -> m + D[parity of m]  -- two integers --
// and the run is VALID for a given incoming m iff no step's exact value falls below 2^23 (there the
// grid is finer) and no state reaches 2^24: m + lo >= 2^23 and m + hi < 2^24, with lo / hi the
// minimum / maximum over the steps of (increment so far + floor(q) / ceil(q)).  Such summaries
// (d0, d1, lo, hi) compose associatively.  For s < 0 the same summary applies to |m| with all four
// numbers negated and lo / hi swapped ("oriented" summaries below).
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define S1_HD __host__ __device__ __forceinline__
#else
#include <cmath>
#include <cstring>
#define S1_HD inline
#endif

namespace repdl_b200 {
namespace s1 {

constexpr int LEAF = 32;                      // elements per leaf (one lane's run)
constexpr int TILE = 32 * LEAF;               // 1024 elements: the 32 leaves of one warp
constexpr int NODE = 32 * TILE;               // 32768 elements
constexpr int LEAVES_PER_NODE = NODE / LEAF;  // 1024
constexpr int TILES_PER_NODE = NODE / TILE;   // 32
constexpr int BIGI = 1 << 29;
constexpr int M_LO = 1 << 23, M_HI = 1 << 24;

S1_HD int f2i(float f)
{
#if defined(__CUDA_ARCH__)
    return __float_as_int(f);
#else
    int i;
    memcpy(&i, &f, 4);
    return i;
#endif
}
S1_HD float i2f(int i)
{
#if defined(__CUDA_ARCH__)
    return __int_as_float(i);
#else
    float f;
    memcpy(&f, &i, 4);
    return f;
#endif
}
S1_HD long long d2ll(double d)
{
#if defined(__CUDA_ARCH__)
    return __double_as_longlong(d);
#else
    long long i;
    memcpy(&i, &d, 8);
    return i;
#endif
}
S1_HD double ll2d(long long i)
{
#if defined(__CUDA_ARCH__)
    return __longlong_as_double(i);
#else
    double d;
    memcpy(&d, &i, 8);
    return d;
#endif
}
// Individually rounded fp32 operations (the host build is compiled without FMA contraction).
S1_HD float mul_rn(float a, float b)
{
#if defined(__CUDA_ARCH__)
    return __fmul_rn(a, b);
#else
    return a * b;
#endif
}
S1_HD float add_rn(float a, float b)
{
#if defined(__CUDA_ARCH__)
    return __fadd_rn(a, b);
#else
    return a + b;
#endif
}
S1_HD float sub_rn(float a, float b)
{
#if defined(__CUDA_ARCH__)
    return __fsub_rn(a, b);
#else
    return a - b;
#endif
}
S1_HD int imin(int a, int b) { return a < b ? a : b; }
S1_HD int imax(int a, int b) { return a > b ? a : b; }
S1_HD int iabs(int a) { return a < 0 ? -a : a; }

struct Summ {
    int d0, d1, lo, hi;  // increments for even / odd incoming m; extreme prefix increments
};

S1_HD Summ summ_identity() { return {0, 0, BIGI, -BIGI}; }  // no steps
S1_HD Summ summ_invalid() { return {0, 0, -BIGI, BIGI}; }
S1_HD bool summ_is_invalid(const Summ &s) { return s.lo <= -(1 << 28) && s.hi >= (1 << 28); }

// a then b (both in the same orientation)
S1_HD Summ summ_compose(const Summ &a, const Summ &b)
{
    if (summ_is_invalid(a) || summ_is_invalid(b)) return summ_invalid();
    Summ r;
    r.d0 = a.d0 + ((a.d0 & 1) ? b.d1 : b.d0);
    r.d1 = a.d1 + (((a.d1 + 1) & 1) ? b.d1 : b.d0);
    const int amin = imin(a.d0, a.d1), amax = imax(a.d0, a.d1);
    r.lo = imin(a.lo, b.lo >= BIGI / 2 ? BIGI : amin + b.lo);
    r.hi = imax(a.hi, b.hi <= -BIGI / 2 ? -BIGI : amax + b.hi);
    if (iabs(r.d0) > (1 << 26) || iabs(r.d1) > (1 << 26)) return summ_invalid();
    return r;
}

// The summary as it applies to |m| of a negative state.
S1_HD Summ summ_orient(const Summ &s, bool neg)
{
    if (!neg || summ_is_invalid(s)) return s;
    return {-s.d0, -s.d1, -s.hi, -s.lo};
}

// Summary of the elements v[0..LEAF) (in order) under binade hypothesis E (exponent field), for a
// positive state.  Hypotheses outside [24, 253] are not summarised (the scale 2^(150-E) must be a
// finite normal float), nor are leaves with an element of 2^22 ulps or more, an infinity or a NaN.
S1_HD Summ leaf_summary(const float *v, int E)
{
    if (E < 24 || E > 253) return summ_invalid();
    const float scale = i2f((277 - E) << 23);  // 2^(150 - E)
    const float MAGIC = 12582912.0f;           // 1.5 * 2^23: q + MAGIC rounds q to an integer
    int d0 = 0, delta = 0;                     // d1 = d0 + delta, |delta| <= 1
    int lo = BIGI, hi = -BIGI;
    bool bad = false, tie_seen = false;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int i = 0; i < LEAF; i++) {
        const float q = mul_rn(v[i], scale);   // exact (power of two) unless it overflows
        bad |= !(fabsf(q) < 4194304.0f);       // |q| >= 2^22, inf or NaN: not summarised
        const float t = add_rn(q, MAGIC);
        int R = f2i(t) - 0x4B400000;           // rint(q), ties to even
        const float d = sub_rn(q, sub_rn(t, MAGIC));  // q - rint(q), exact, in [-0.5, 0.5]
        // The step is modelled correctly iff its exact value m + q is not below 2^23 (there the
        // grid is finer), i.e. iff m + D_before + floor(q) >= 2^23 (m and D are integers).  For a
        // negative state the same condition reads |m| - (D_before + ceil(q)) >= 2^23, so `hi`
        // tracks D_before + ceil(q): it bounds the reachable states from above (within one unit)
        // and becomes the exact lower bound when the summary is negated.
        const int fl = d0 + R + (f2i(d) >> 31);  // D_before + floor(q) (d = -0 gives a bound one unit too careful)
        lo = imin(lo, fl);
        hi = imax(hi, fl + (d != 0.0f ? 1 : 0));  // D_before + ceil(q)
        if (fabsf(d) == 0.5f && !bad) {
            // exact tie: the result is the even one of m+n, m+n+1 with n = floor(q)
            const int n = d > 0.0f ? R : R - 1;
            const int inc0 = n + ((d0 + n) & 1);
            const int inc1 = n + ((1 + d0 + delta + n) & 1);
            delta += inc1 - inc0;
            R = inc0;
            tie_seen = true;
        }
        d0 += R;
    }
    if (bad) return summ_invalid();
    // after a tie the odd-parity track may run one off the even one: widen by 1 to cover both
    const int margin = tie_seen ? 1 : 0;
    return {d0, d0 + delta, lo - margin, hi + margin};
}

// ------------------------------------------------------------------------------------------------
// Prediction.  The exact chain state is only known to the walker; everything that is prepared in
// parallel works from an fp64 prefix sum p of the elements (the "predicted state") and an estimate
// R of how far the fp32 chain may have drifted from it.
// ------------------------------------------------------------------------------------------------

// Exponent field (1..254) a float of magnitude |a| would have; 0 for zero / tiny, 255 for huge.
S1_HD int exp_field_of(double a)
{
    const long long b = d2ll(a) & 0x7FFFFFFFFFFFFFFFll;
    const int de = (int)(b >> 52) - 1023 + 127;
    return de < 0 ? 0 : (de > 255 ? 255 : de);
}
S1_HD double pow2(int e) { return ll2d((long long)(e + 1023) << 52); }  // 2^e, -1022 <= e <= 1023

// The hypothesis (sign bit << 8 | exponent field) under which a leaf that the chain is predicted
// to enter with state p is summarised.
S1_HD int hyp_sign_exp(double p) { return (p < 0.0 ? 256 : 0) | exp_field_of(p); }

// Variance that one node adds to the drift of the chain: NODE roundings, each uniform within half
// an ulp of a state of magnitude a.
S1_HD double drift_variance(double a)
{
    int E = exp_field_of(a);
    E = E < 1 ? 1 : (E > 254 ? 254 : E);
    const double u = pow2(E - 150);
    return (double)NODE * u * u * (1.0 / 12.0);
}
#ifndef REPDL_SUM1D_SIGMAS
#define REPDL_SUM1D_SIGMAS 3.5
#endif
constexpr double DRIFT_SIGMAS = REPDL_SUM1D_SIGMAS;

enum LeafClass { C_ROBUST = 0, C_SOFT = 1, C_HARD = 2 };

// How a leaf with positive-orientation summary `sm` under hypothesis `sek` (hyp_sign_exp(p)) is
// expected to behave: C_ROBUST -- valid for every state within rabs of the prediction p;
// C_SOFT -- valid for p itself; C_HARD -- not even that.
S1_HD int classify_leaf(const Summ &sm, int sek, double p, double rabs)
{
    if (summ_is_invalid(sm)) return C_HARD;
    const int E = sek & 255;
    const bool neg = (sek & 256) != 0;
    const double sc = pow2(150 - E);  // E in [24, 253] here
    const double m = (neg ? -p : p) * sc;
    const double lo = neg ? -(double)sm.hi : (double)sm.lo;
    const double hi = neg ? -(double)sm.lo : (double)sm.hi;
    const double ru = rabs * sc + 2.0;
    if (m + lo - ru >= (double)M_LO && m + hi + ru < (double)M_HI) return C_ROBUST;
    if (m + lo >= (double)M_LO && m + hi < (double)M_HI) return C_SOFT;
    return C_HARD;
}

// ------------------------------------------------------------------------------------------------
// The item stream the walker consumes.  Items are in chain order; each covers `len` leaves from
// leaf `start` on.
//   K_RUN      leaves that are all C_ROBUST under one hypothesis, composed; if the summary is not
//              valid for the exact state (a prediction that was off by more than the margin) the
//              span is walked with real adds
//   K_SOFT     two or more C_SOFT leaves under one hypothesis, composed; valid -> applied and the
//              next `skip` items (its leaves, one K_LEAF each) are skipped; else the walker goes on
//              to those
//   K_LEAF     one C_SOFT leaf: summary if valid, else 32 real adds
//   K_HARD     one leaf that is walked with 32 real adds
//   K_RAWSPAN  a span that is walked with real adds (a node that no longer fitted into the item
//              buffer)
// ------------------------------------------------------------------------------------------------
enum ItemKind { K_RUN = 0, K_SOFT = 1, K_LEAF = 2, K_HARD = 3, K_RAWSPAN = 4 };

struct alignas(16) Item {
    int d0, d1, lo, hi;  // oriented summary (K_RUN, K_SOFT, K_LEAF)
    int sek;             // hypothesis: sign << 8 | exponent field
    int kind_skip;       // kind | skip << 8
    int start, len;      // in leaves
};
static_assert(sizeof(Item) == 32, "two 16-byte words");

S1_HD Item make_item(int kind, const Summ &pos, int sek, int skip, int start, int len)
{
    const Summ o = summ_orient(pos, (sek & 256) != 0);
    return {o.d0, o.d1, o.lo, o.hi, sek, kind | (skip << 8), start, len};
}

// Applies a summarising item to the exact state (as bits) if it is valid for it.
S1_HD bool item_apply(int &bits, const Item &it)
{
    if (((bits >> 23) & 0x1FF) != it.sek) return false;
    const int m = (bits & 0x7FFFFF) | 0x800000;
    if (m + it.lo < M_LO || m + it.hi >= M_HI) return false;
    bits += (bits & 1) ? it.d1 : it.d0;  // |m| stays inside [2^23, 2^24): only the mantissa field moves
    return true;
}

// Per-leaf code inside a node: class << 9 | hypothesis.
S1_HD int leaf_code(int cls, int sek) { return (cls << 9) | sek; }
S1_HD int code_class(int code) { return code >> 9; }
S1_HD int code_sek(int code) { return code & 0x1FF; }

// First leaf of a run of equal codes (robust and soft leaves form runs; a hard leaf stands alone).
S1_HD bool leaf_is_head(const unsigned short *code, int i) { return i == 0 || code[i - 1] != code[i]; }

// Number of items leaf i of a node contributes.
S1_HD int leaf_item_count(const unsigned short *code, int i)
{
    const int c = code[i], cls = code_class(c);
    if (cls == C_HARD) return 1;
    const bool head = leaf_is_head(code, i);
    if (cls == C_ROBUST) return head ? 1 : 0;
    const bool longer = i + 1 < LEAVES_PER_NODE && code[i + 1] == c;
    return 1 + ((head && longer) ? 1 : 0);
}

// Writes the items of leaf i (leaf_item_count(code, i) of them) to out[0..).  `summ` holds the
// positive-orientation summaries of the node's leaves, `leaf0` is the node's first leaf.
S1_HD void leaf_emit_items(const unsigned short *code, const Summ *summ, int i, int leaf0, Item *out)
{
    const int c = code[i], cls = code_class(c), sek = code_sek(c);
    if (cls == C_HARD) {
        out[0] = make_item(K_HARD, summ_invalid(), sek, 0, leaf0 + i, 1);
        return;
    }
    const bool head = leaf_is_head(code, i);
    if (cls == C_ROBUST && !head) return;
    int len = 1;
    Summ acc = summ[i];
    if (head) {
        while (i + len < LEAVES_PER_NODE && code[i + len] == c) {
            acc = summ_compose(acc, summ[i + len]);
            len++;
        }
    }
    if (cls == C_ROBUST) {
        out[0] = make_item(K_RUN, acc, sek, 0, leaf0 + i, len);
        return;
    }
    int k = 0;
    if (head && len > 1) out[k++] = make_item(K_SOFT, acc, sek, len, leaf0 + i, len);
    out[k] = make_item(K_LEAF, summ[i], sek, 0, leaf0 + i, 1);
}

// Item buffer capacity for a chain of nnodes nodes.
S1_HD long long item_capacity(long long nnodes) { return 24 * nnodes + 32768; }

}  // namespace s1
}  // namespace repdl_b200
