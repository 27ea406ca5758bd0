// sum1d: ONE strict left-to-right fp32 chain over n elements (microsoft/RepDL
// backend/cpu/summation.cpp:12-20: `sum += I[i]` from +0, then `factor * sum`), reproduced bit for
// bit but not walked element by element.
//
// Why a chain can be summarised.  While the running sum s stays inside one binade (exponent field
// E, ulp u = 2^(E-150)), s = m*u with an integer 2^23 <= |m| < 2^24, and a rounded fp32 add of
// x = q*u gives exactly m' = m + rint(q), rint = round-half-even; on an exact tie (q = n + 1/2) the
// result is whichever of m+n, m+n+1 is even, i.e. it depends on the parity of m.  So, for a fixed
// binade hypothesis E, a run of elements acts on m as  m -> m + D[parity of m]  -- two integers --
// and the run is VALID for a given incoming m iff no step's exact value falls below 2^23 (there the
// grid is finer) and no state reaches 2^24: m + lo >= 2^23 and m + hi < 2^24, with lo / hi the
// minimum / maximum over the steps of (increment so far + floor(q) / ceil(q)).  Such
// summaries (D0, D1, lo, hi) compose associatively, so they can be built by a tree in parallel.
// (For s < 0 the same summary applies to |m| with all four numbers negated and lo/hi swapped.)
//
// Pipeline (all deterministic, no atomics):
//   1. node_sum_kernel      fp64 sum of every node of 32768 elements (only used to PREDICT)
//   2. node_scan_kernel     exclusive scan of those sums -> predicted chain state at each node
//                           start, and from it two binade hypotheses per node: the predicted
//                           binade and its nearer neighbour
//   3. summarise_kernel     per node: leaf summaries (32 elements per lane) under both hypotheses,
//                           composed (in order) to one summary per node
//   4. walk_kernel          one thread-block cluster; warp 0 of its first CTA carries the exact
//                           fp32 state through the nodes: 32 node summaries are composed by a warp
//                           scan and applied in one step when they are valid for the exact state;
//                           the first node that is not valid (a real binade change, a wrong
//                           prediction, a huge element, inf/NaN) is opened: the cluster's warps stage
//                           its 32 tiles in (distributed) shared memory and summarise them, one tile
//                           and binade per warp, under the exact binade and its nearer neighbour, warp 0 walks the
//                           tiles the same way, an invalid tile has its 32 leaves summarised on the
//                           fly, and an invalid leaf is finally walked with 32 real fp32 adds.
//                           After an opened child the scan is not redone: its prefix increments are
//                           re-anchored on the new exact state (valid while binade, sign and --
//                           where ties follow -- parity are unchanged).
// A wrong prediction therefore costs time, never bits: every summary is applied only after its
// validity has been checked against the exact state, and everything else is real fp32 addition.
// Elements past n are treated as +0.0f, which never changes a chain that started at +0 (such a
// chain cannot hold -0).
#include "common.cuh"

#include <cooperative_groups.h>

namespace repdl_b200 {
namespace {

constexpr int LEAF = 32;            // elements per lane
constexpr int TILE = 32 * LEAF;     // 1024 elements per warp tile
constexpr int NODE = 32 * TILE;     // 32768 elements per node
constexpr int BIGI = 1 << 29;
constexpr int M_LO = 1 << 23, M_HI = 1 << 24;

struct Summ {
    int d0, d1, lo, hi;  // increments for even / odd incoming m; extreme prefix increments
};

__device__ __forceinline__ Summ summ_identity() { return {0, 0, BIGI, -BIGI}; }  // no steps
__device__ __forceinline__ Summ summ_invalid() { return {0, 0, -BIGI, BIGI}; }
__device__ __forceinline__ bool summ_is_invalid(const Summ &s)
{
    return s.lo <= -(1 << 28) && s.hi >= (1 << 28);
}

// a then b
__device__ __forceinline__ Summ summ_compose(const Summ &a, const Summ &b)
{
    if (summ_is_invalid(a) || summ_is_invalid(b)) return summ_invalid();
    Summ r;
    r.d0 = a.d0 + ((a.d0 & 1) ? b.d1 : b.d0);
    r.d1 = a.d1 + (((a.d1 + 1) & 1) ? b.d1 : b.d0);
    const int amin = min(a.d0, a.d1), amax = max(a.d0, a.d1);
    r.lo = min(a.lo, b.lo >= BIGI / 2 ? BIGI : amin + b.lo);
    r.hi = max(a.hi, b.hi <= -BIGI / 2 ? -BIGI : amax + b.hi);
    if (abs(r.d0) > (1 << 26) || abs(r.d1) > (1 << 26)) return summ_invalid();
    return r;
}

__device__ __forceinline__ Summ shfl_up_summ(const Summ &s, int delta)
{
    return {__shfl_up_sync(0xffffffffu, s.d0, delta), __shfl_up_sync(0xffffffffu, s.d1, delta),
            __shfl_up_sync(0xffffffffu, s.lo, delta), __shfl_up_sync(0xffffffffu, s.hi, delta)};
}

// Summary of the elements v[0..LEAF) (in order) under binade hypothesis E (exponent field).
// Hypotheses outside [24, 253] are not summarised (the scale 2^(150-E) must be a finite float).
__device__ __forceinline__ Summ leaf_summary(const float (&v)[LEAF], int E, bool *had_tie = nullptr)
{
    if (had_tie) *had_tie = false;
    if (E < 24 || E > 253) return summ_invalid();
    const float scale = __int_as_float((277 - E) << 23);  // 2^(150 - E)
    const float MAGIC = 12582912.0f;                       // 1.5 * 2^23: q + MAGIC rounds q to an integer
    int d0 = 0, delta = 0;                                 // d1 = d0 + delta, |delta| <= 1
    int lo = BIGI, hi = -BIGI;
    bool bad = false, tie_seen = false;
#pragma unroll
    for (int i = 0; i < LEAF; i++) {
        const float q = __fmul_rn(v[i], scale);            // exact (power of two) unless it overflows
        bad |= !(fabsf(q) < 4194304.0f);                   // |q| >= 2^22, inf or NaN: not summarised
        const float t = __fadd_rn(q, MAGIC);
        int R = __float_as_int(t) - 0x4B400000;            // rint(q), ties to even
        const float d = __fsub_rn(q, __fsub_rn(t, MAGIC)); // q - rint(q), exact, in [-0.5, 0.5]
        // The step is modelled correctly iff its exact value m + q is not below 2^23 (there the
        // grid is finer), i.e. iff m + D_before + floor(q) >= 2^23 (m and D are integers).  For a
        // negative state the same condition reads |m| - (D_before + ceil(q)) >= 2^23, so `hi`
        // tracks D_before + ceil(q): it bounds the reachable states from above (within one unit)
        // and becomes the exact lower bound when the summary is negated.
        const int fl = d0 + R + (__float_as_int(d) >> 31);  // D_before + floor(q) (an element of -0.0f gives d = -0 and a bound one unit too careful)
        lo = min(lo, fl);
        hi = max(hi, fl + (d != 0.0f ? 1 : 0));             // D_before + ceil(q)
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
    if (had_tie) *had_tie = tie_seen;
    if (bad) return summ_invalid();
    // after a tie the odd-parity track may run one off the even one: widen by 1 to cover both
    const int margin = tie_seen ? 1 : 0;
    return {d0, d0 + delta, lo - margin, hi + margin};
}

__device__ __forceinline__ int exp_field(float s) { return (__float_as_int(s) >> 23) & 0xFF; }

// State s (binade E >= 1, so |m| in [2^23, 2^24)) plus a signed increment of |m| -> new state.
__device__ __forceinline__ float apply_inc(float s, int inc)
{
    const unsigned b = (unsigned)__float_as_int(s);
    const int m = (int)((b & 0x7FFFFFu) | 0x800000u) + inc;  // stays in [2^23, 2^24) when valid
    return __int_as_float((int)((b & 0xFF800000u) | ((unsigned)m & 0x7FFFFFu)));
}

// Scan context of one binade hypothesis over the 32 children of a level (one child per lane).
struct Ctx {
    Summ mine;   // this lane's child under binade E (positive orientation; identity before pos0)
    int c0, c1;  // increments of |m| from pos0 to this lane's start, for even / odd m at pos0
    int t0, t1;  // the same through the last child
    unsigned tiemask, invmask;
    int E, pos0;
};

__device__ __forceinline__ void ctx_scan(Ctx &cx, int pos)
{
    const int lane = threadIdx.x & 31;
    if (lane < pos) cx.mine = summ_identity();
    Summ incl = cx.mine;
#pragma unroll
    for (int dlt = 1; dlt < 32; dlt <<= 1) {
        Summ up = shfl_up_summ(incl, dlt);
        if (lane >= dlt) incl = summ_compose(up, incl);
    }
    cx.c0 = __shfl_up_sync(0xffffffffu, incl.d0, 1);
    cx.c1 = __shfl_up_sync(0xffffffffu, incl.d1, 1);
    if (lane <= pos) cx.c0 = cx.c1 = 0;
    cx.t0 = __shfl_sync(0xffffffffu, incl.d0, 31);
    cx.t1 = __shfl_sync(0xffffffffu, incl.d1, 31);
    cx.tiemask = __ballot_sync(0xffffffffu, lane >= pos && cx.mine.d0 != cx.mine.d1);
    cx.invmask = __ballot_sync(0xffffffffu, lane >= pos && summ_is_invalid(cx.mine));
    cx.pos0 = pos;
}

// One level of the walk, run by one full warp.  `count` children (<= 32), child c owned by lane c
// (lanes >= count must supply identity summaries).
//   hypE0/hypE1      the two binades for which summaries exist up front;
//   getH(k)          this lane's summary under hypothesis k (positive orientation);
//   getE(E)          this lane's summary under an arbitrary binade E, or invalid if the level
//                    cannot make one;
//   open(j, s)       the exact state after child j entered with state s (warp-uniform call).
// Returns the exact state after all children.  The two contexts are scanned once; after an opened
// child the prefix increments of the context that matches the new binade are re-anchored on the
// new exact state, which is valid while no child with an invalid summary has been passed and --
// where ties follow -- a start parity exists that reproduces the actual parity.
template <class GetH, class GetE, class Open>
__device__ __forceinline__ float walk_level(float s, int count, int hypE0, int hypE1, GetH getH,
                                            GetE getE, Open open, int &opens)
{
    const int lane = threadIdx.x & 31;
    Ctx cxA, cxB;  // kept as two named objects so that they stay in registers
    cxA.mine = lane < count ? getH(0) : summ_identity();
    cxA.E = hypE0;
    ctx_scan(cxA, 0);
    cxB.mine = lane < count ? getH(1) : summ_identity();
    cxB.E = hypE1;
    ctx_scan(cxB, 0);
    int pos = 0;
    bool done = false;
    // one attempt to advance with context c (which matches the binade of s); opens one child
    auto step = [&](Ctx &c) {
        const bool neg = __float_as_int(s) < 0;
        const int m = (int)(((unsigned)__float_as_int(s) & 0x7FFFFFu) | 0x800000u);
        const unsigned from_pos = 0xFFFFFFFFu << pos;
        // pick the start parity p whose track has the actual parity at pos
        int p = -1;
        if ((c.invmask & (0xFFFFFFFFu << c.pos0) & ~from_pos) == 0u) {
            const int a0 = __shfl_sync(0xffffffffu, c.c0, pos), a1 = __shfl_sync(0xffffffffu, c.c1, pos);
            if (((a0 ^ m) & 1) == 0)
                p = 0;
            else if ((((1 + a1) ^ m) & 1) == 0)
                p = 1;
            else if ((c.tiemask & from_pos) == 0u)
                p = 0;  // no tie ahead: the increments do not depend on parity
        }
        if (p < 0) {
            ctx_scan(c, pos);
            p = m & 1;
        }
        const int cl = p ? c.c1 : c.c0;
        const int cpos = __shfl_sync(0xffffffffu, cl, pos);
        const int m_in = m + (neg ? -(cl - cpos) : (cl - cpos));  // |m| entering this lane's child
        const int wlo = neg ? -c.mine.hi : c.mine.lo, whi = neg ? -c.mine.lo : c.mine.hi;
        bool ok = true;
        if (lane >= pos && lane < count) {
            ok = !summ_is_invalid(c.mine) &&
                 ((c.invmask & (0xFFFFFFFFu << c.pos0) & ~(0xFFFFFFFFu << lane)) == 0u) &&
                 (m_in + wlo >= M_LO) && (m_in + whi < M_HI);
        }
        const unsigned badmask = __ballot_sync(0xffffffffu, !ok);
        if (badmask == 0u) {
            const int tot = (p ? c.t1 : c.t0) - cpos;
            s = apply_inc(s, neg ? -tot : tot);
            done = true;
            return;
        }
        const int j = __ffs((int)badmask) - 1;
        if (j > pos) s = apply_inc(s, __shfl_sync(0xffffffffu, m_in, j) - m);
        s = open(j, s);
        opens++;
        pos = j + 1;
    };
    while (pos < count && !done) {
        const int E = exp_field(s);
        if (E == cxA.E) {
            step(cxA);
        } else {
            if (E != cxB.E) {
                // a binade nobody prepared: make a context for it in slot B, from pos on
                cxB.mine = (lane >= pos && lane < count)
                               ? ((E < 24 || E > 253) ? summ_invalid() : getE(E))
                               : summ_identity();
                cxB.E = E;
                ctx_scan(cxB, pos);
            }
            step(cxB);
        }
    }
    return s;
}

// ------------------------------------------------------------------------------------------------
// The leaf level of the walk uses a lighter algebra: a leaf that contains an exact tie is simply
// treated like an invalid one (it is walked with real adds), so a leaf is (d, lo, hi) with no
// parity tracks and composition is an add and two min/max.  Ties are rare (about 1 step in 10^4),
// and only leaves of opened tiles pass through here, so this costs a handful of extra leaf walks.
// ------------------------------------------------------------------------------------------------
// Cycle counters of the walker warp, kept in the scratch header for diagnostics.
// Cycle counters of the walker (diagnostics in the scratch header); compiled out unless asked for,
// since reading the clock a few times per opened leaf is itself a measurable part of the walk.
#ifndef REPDL_SUM1D_CLOCKS
#define REPDL_SUM1D_CLOCKS 0
#endif
__device__ __forceinline__ long long walk_clock()
{
#if REPDL_SUM1D_CLOCKS
    return clock64();
#else
    return 0;
#endif
}

struct WalkClock {
    long long prepare, tile_scan, leaf_steps, raw, rebuild, load;
};

struct LeafCtx {
    int lo, hi;   // this lane's leaf: extreme (increment so far + floor/ceil(q)), relative to its start
    int c, tot;   // increment from pos0 to this lane's start / through the last leaf
    unsigned invmask;
    int E, pos0;
};

__device__ __forceinline__ void leaf_ctx_build(LeafCtx &cx, const float (&v)[LEAF], int E, int pos)
{
    const int lane = threadIdx.x & 31;
    const bool usable = E >= 24 && E <= 253;
    const float scale = __int_as_float((277 - (usable ? E : 127)) << 23);  // 2^(150 - E)
    const float MAGIC = 12582912.0f;
    int d = 0, lo = BIGI, hi = -BIGI;
    bool bad = !usable;
#pragma unroll
    for (int i = 0; i < LEAF; i++) {
        const float q = __fmul_rn(v[i], scale);
        const float t = __fadd_rn(q, MAGIC);
        const int R = __float_as_int(t) - 0x4B400000;
        const float r = __fsub_rn(q, __fsub_rn(t, MAGIC));       // q - rint(q)
        bad |= !(fabsf(q) < 4194304.0f) | (fabsf(r) == 0.5f);     // huge, inf, NaN or an exact tie
        const int fl = d + R + (__float_as_int(r) >> 31);
        lo = min(lo, fl);
        hi = max(hi, fl + (r != 0.0f ? 1 : 0));
        d += R;
    }
    if (lane < pos) d = 0, lo = BIGI, hi = -BIGI, bad = false;
    cx.lo = lo, cx.hi = hi;
    cx.invmask = __ballot_sync(0xffffffffu, bad);
    // inclusive prefix sum of d (values past an invalid leaf are never used before a rebuild)
    int incl = bad ? 0 : d;
#pragma unroll
    for (int dlt = 1; dlt < 32; dlt <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, dlt);
        if (lane >= dlt) incl += up;
    }
    cx.c = __shfl_up_sync(0xffffffffu, incl, 1);
    if (lane == 0) cx.c = 0;
    cx.tot = __shfl_sync(0xffffffffu, incl, 31);
    cx.E = E, cx.pos0 = pos;
}

// The same context made from a full leaf summary that is already at hand (whole tile, pos = 0).
__device__ __forceinline__ void leaf_ctx_from_summary(LeafCtx &cx, const Summ &sm, bool tie, int E)
{
    const int lane = threadIdx.x & 31;
    const bool bad = tie || summ_is_invalid(sm);
    cx.lo = sm.lo, cx.hi = sm.hi;
    cx.invmask = __ballot_sync(0xffffffffu, bad);
    int incl = bad ? 0 : sm.d0;
#pragma unroll
    for (int dlt = 1; dlt < 32; dlt <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, dlt);
        if (lane >= dlt) incl += up;
    }
    cx.c = __shfl_up_sync(0xffffffffu, incl, 1);
    if (lane == 0) cx.c = 0;
    cx.tot = __shfl_sync(0xffffffffu, incl, 31);
    cx.E = E, cx.pos0 = 0;
}

// Walks the 32 leaves (lane-owned runs v) of one tile from exact state s, starting from the two
// prepared contexts.
__device__ __forceinline__ float walk_leaves(float s, const float (&v)[LEAF], LeafCtx cxA, LeafCtx cxB,
                                             int &opens, WalkClock &clk)
{
    const int lane = threadIdx.x & 31;
    const long long t_enter = walk_clock();
    int pos = 0;
    bool done = false;
    auto step = [&](LeafCtx &c) {
        const bool neg = __float_as_int(s) < 0;
        const int m = (int)(((unsigned)__float_as_int(s) & 0x7FFFFFu) | 0x800000u);
        // c.c is a plain prefix sum in which an invalid leaf counts as 0, so the difference
        // c.c - cpos is exact for every lane with no invalid leaf in [pos, lane): invalid leaves
        // that have already been passed cancel out and never force a rebuild
        const int cpos = __shfl_sync(0xffffffffu, c.c, pos);
        const int m_in = m + (neg ? -(c.c - cpos) : (c.c - cpos));
        const int wlo = neg ? -c.hi : c.lo, whi = neg ? -c.lo : c.hi;
        const unsigned inv_ahead = c.invmask & (0xFFFFFFFFu << pos);
        const bool before_inv = (inv_ahead & ~(0xFFFFFFFFu << lane)) != 0u;
        const bool ok = lane < pos || lane < c.pos0 ||
                        (!((c.invmask >> lane) & 1u) && !before_inv && (m_in + wlo >= M_LO) &&
                         (m_in + whi < M_HI));
        const unsigned badmask = __ballot_sync(0xffffffffu, !ok);
        if (badmask == 0u) {
            const int tot = c.tot - cpos;
            s = apply_inc(s, neg ? -tot : tot);
            done = true;
            return;
        }
        const int j = __ffs((int)badmask) - 1;
        if (j > pos) s = apply_inc(s, __shfl_sync(0xffffffffu, m_in, j) - m);
        // open leaf j: 32 real fp32 adds by its owner
        const long long t0 = walk_clock();
        float r = s;
        if (lane == j) {
#pragma unroll
            for (int i = 0; i < LEAF; i++) r = __fadd_rn(r, v[i]);
        }
        s = __shfl_sync(0xffffffffu, r, j);
        clk.raw += walk_clock() - t0;
        opens++;
        pos = j + 1;
    };
#ifndef REPDL_SUM1D_RAW3
#define REPDL_SUM1D_RAW3 3
#endif
    int raw_run = 0;  // leaves walked with real adds in a row because the state sat in a third binade
    while (pos < 32 && !done) {
        const int E = exp_field(s);
        if (E == cxA.E) {
            step(cxA);
            raw_run = 0;
        } else if (E == cxB.E) {
            step(cxB);
            raw_run = 0;
        } else if (raw_run < REPDL_SUM1D_RAW3) {
            // A third binade (the state is crossing several binades, typically near zero): the next
            // leaf's 32 real adds cost a fraction of a new context, and the state has often moved on
            // to a prepared binade after them.
            const long long t0 = walk_clock();
            float r = s;
            if (lane == pos) {
#pragma unroll
                for (int i = 0; i < LEAF; i++) r = __fadd_rn(r, v[i]);
            }
            s = __shfl_sync(0xffffffffu, r, pos);
            clk.raw += walk_clock() - t0;
            opens++;
            pos++;
            raw_run++;
        } else {
            const long long t0 = walk_clock();
            leaf_ctx_build(cxB, v, E, pos);
            clk.rebuild += walk_clock() - t0;
            step(cxB);
            raw_run = 0;
        }
    }
    clk.leaf_steps += walk_clock() - t_enter;
    return s;
}

// Loads lane-owned run [base + 32*lane, +32) of the chain; elements at or past n read as +0.
__device__ __forceinline__ void load_leaf(const float *__restrict__ x, int64_t n, int64_t base,
                                          bool vec, float (&v)[LEAF])
{
    const int lane = threadIdx.x & 31;
    const int64_t e0 = base + (int64_t)lane * LEAF;
    if (vec && e0 + LEAF <= n) {
        const float4 *p = reinterpret_cast<const float4 *>(x + e0);
#pragma unroll
        for (int i = 0; i < LEAF / 4; i++) {
            float4 t = __ldg(p + i);
            v[4 * i + 0] = t.x, v[4 * i + 1] = t.y, v[4 * i + 2] = t.z, v[4 * i + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < LEAF; i++) v[i] = (e0 + i < n) ? __ldg(x + e0 + i) : 0.0f;
    }
}

// ---------------------------------------------------------------------------------------------
// 1. fp64 sum per node (prediction only)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
node_sum_kernel(const float *__restrict__ x, int64_t n, double *__restrict__ node_sum, int vec)
{
    __shared__ double part[8];
    const int64_t base = (int64_t)blockIdx.x * NODE;
    const int t = threadIdx.x;
    double acc = 0.0;
    if (vec && base + NODE <= n) {
        const float4 *p = reinterpret_cast<const float4 *>(x + base);
#pragma unroll 8
        for (int i = t; i < NODE / 4; i += 256) {
            float4 v = __ldg(p + i);
            acc += (double)v.x + (double)v.y + (double)v.z + (double)v.w;
        }
    } else {
        for (int i = t; i < NODE; i += 256)
            if (base + i < n) acc += (double)__ldg(x + base + i);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, d);
    if ((t & 31) == 0) part[t >> 5] = acc;
    __syncthreads();
    if (t == 0) {
        double s = 0.0;
        for (int w = 0; w < 8; w++) s += part[w];
        node_sum[blockIdx.x] = s;
    }
}

// ---------------------------------------------------------------------------------------------
// 2. exclusive scan of the node sums (one CTA) -> two binade hypotheses per node
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int2 hypotheses_for(double pred)
{
    // exponent field a float of magnitude |pred| would have, and the neighbour nearer in log scale
    const double a = fabs(pred);
    int e = 0, e2 = 0;
    if (a > 0.0 && a < 3.0e38) {
        const long long b = __double_as_longlong(a);
        const int de = (int)((b >> 52) & 0x7FF) - 1023;  // floor(log2 a)
        e = min(max(de + 127, 1), 254);
        const bool upper_half = ((b >> 51) & 1) != 0;     // mantissa >= 1.5
        e2 = min(max(e + (upper_half ? 1 : -1), 1), 254);
    }
    return make_int2(e, e2);
}

__global__ void __launch_bounds__(1024)
node_scan_kernel(const double *__restrict__ node_sum, int nnodes, int2 *__restrict__ hyp)
{
    __shared__ double chunk_total[1024];
    const int t = threadIdx.x;
    const int per = (nnodes + 1023) / 1024;
    const int lo = t * per, hi = min(lo + per, nnodes);
    double s = 0.0;
    for (int i = lo; i < hi; i++) s += node_sum[i];
    chunk_total[t] = s;
    __syncthreads();
    if (t == 0) {
        double run = 0.0;
        for (int i = 0; i < 1024; i++) {
            double c = chunk_total[i];
            chunk_total[i] = run;
            run += c;
        }
    }
    __syncthreads();
    double run = chunk_total[t];
    for (int i = lo; i < hi; i++) {
        hyp[i] = hypotheses_for(run);
        run += node_sum[i];
    }
}

// ---------------------------------------------------------------------------------------------
// 3. node summaries under both hypotheses
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ Summ warp_reduce_summ(Summ s)
{
    // ordered reduction: lane 0 ends with s_0 o s_1 o ... o s_31
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int dlt = 1; dlt < 32; dlt <<= 1) {
        Summ other = {__shfl_down_sync(0xffffffffu, s.d0, dlt), __shfl_down_sync(0xffffffffu, s.d1, dlt),
                      __shfl_down_sync(0xffffffffu, s.lo, dlt), __shfl_down_sync(0xffffffffu, s.hi, dlt)};
        if ((lane & (2 * dlt - 1)) == 0) s = summ_compose(s, other);
    }
    return s;
}

__global__ void __launch_bounds__(256)
summarise_kernel(const float *__restrict__ x, int64_t n, const int2 *__restrict__ hyp,
                 int4 *__restrict__ nodeA, int4 *__restrict__ nodeB, int vec)
{
    __shared__ Summ sA[32], sB[32];
    const int node = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int2 h = hyp[node];
    for (int tl = warp; tl < 32; tl += 8) {
        float v[LEAF];
        load_leaf(x, n, (int64_t)node * NODE + (int64_t)tl * TILE, vec != 0, v);
        Summ a = warp_reduce_summ(leaf_summary(v, h.x));
        Summ b = warp_reduce_summ(leaf_summary(v, h.y));
        if (lane == 0) {
            sA[tl] = a;
            sB[tl] = b;
        }
    }
    __syncthreads();
    if (warp == 0) {
        Summ a = warp_reduce_summ(sA[lane]);
        Summ b = warp_reduce_summ(sB[lane]);
        if (lane == 0) {
            nodeA[node] = make_int4(a.d0, a.d1, a.lo, a.hi);
            nodeB[node] = make_int4(b.d0, b.d1, b.lo, b.hi);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// 4. the walk: one CTA; warp 0 walks, all warps prepare an opened node
// ---------------------------------------------------------------------------------------------
// CTAs (SMs) that prepare an opened node together: the largest portable cluster.  Measured on B200 for
// the 2^28-element chain: 2 CTAs 23.1 ms, 4 CTAs 18.5 ms, 8 CTAs 17.0 ms, 16 (non-portable) 16.8 ms.
constexpr int WALK_CLUSTER = 8;
constexpr int WALK_THREADS = 64 * 32 / WALK_CLUSTER;  // one warp per (tile, binade) job of a CTA
constexpr int TPC = 32 / WALK_CLUSTER;  // tiles of a node per CTA: one (tile, binade) job per warp
static_assert(TPC * 2 == WALK_THREADS / 32, "one job per warp");
constexpr int RUN_PITCH = 36;  // floats per lane-run in shared memory: LDS.128 without bank conflicts
struct WalkShared {
    float raw[TPC][32 * RUN_PITCH];  // this CTA's tiles of the opened node
    Summ tile[2][TPC];               // their summaries under the two binades of `e`
    int leaf_lo[2][TPC][32], leaf_hi[2][TPC][32], leaf_c[2][TPC][32];  // leaf contexts, [binade][tile][lane]
    int leaf_tot[2][TPC];
    unsigned leaf_inv[2][TPC];
    int e[2];                        // (CTA 0 only) binades to summarise under
    int cmd;                         // (CTA 0 only) node to open, or -1: finished
};
constexpr int WALK_SMEM_BYTES = (int)sizeof(WalkShared);

// Every warp of every CTA of the cluster: one tile of node nd under one of the two binades that the
// walker left in CTA 0's shared memory (`ctl`).  Tile tl of the node lives in CTA tl / TPC.
__device__ __forceinline__ void prepare_node(WalkShared &sh, const WalkShared *ctl, int rank,
                                             const float *__restrict__ x, int64_t n, int nd, bool vec)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tl = warp >> 1, h = warp & 1;
    const int E = ctl->e[h];
    float v[LEAF];
    load_leaf(x, n, (int64_t)nd * NODE + (int64_t)(rank * TPC + tl) * TILE, vec, v);
    if (h == 0) {
        float4 *dst = reinterpret_cast<float4 *>(&sh.raw[tl][lane * RUN_PITCH]);
#pragma unroll
        for (int i = 0; i < LEAF / 4; i++)
            dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    }
    bool tie;
    const Summ leaf = leaf_summary(v, E, &tie);
    LeafCtx cx;
    leaf_ctx_from_summary(cx, leaf, tie, E);
    sh.leaf_lo[h][tl][lane] = cx.lo;
    sh.leaf_hi[h][tl][lane] = cx.hi;
    sh.leaf_c[h][tl][lane] = cx.c;
    const Summ t = warp_reduce_summ(leaf);
    if (lane == 0) {
        sh.tile[h][tl] = t;
        sh.leaf_tot[h][tl] = cx.tot;
        sh.leaf_inv[h][tl] = cx.invmask;
    }
}

// Launched as ONE cluster of WALK_CLUSTER CTAs.  Warp 0 of CTA 0 carries the exact state; everything
// else only helps to prepare opened nodes.  The CTAs meet at the cluster's hardware barrier (no
// spinning on memory): A -- a command is posted; B -- the node is prepared.  Between B and the next A
// the walker reads the other CTAs' shared memory (distributed shared memory), which nobody writes then.
__global__ void __launch_bounds__(WALK_THREADS, 1)
walk_kernel(const float *__restrict__ x, int64_t n, int nnodes, const int2 *__restrict__ hyp,
            const int4 *__restrict__ nodeA, const int4 *__restrict__ nodeB, float factor,
            float *__restrict__ out, int vec, int *__restrict__ stats)
{
    namespace cg = cooperative_groups;
    extern __shared__ __align__(16) unsigned char walk_smem[];
    WalkShared &sh = *reinterpret_cast<WalkShared *>(walk_smem);
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const WalkShared *ctl = cluster.map_shared_rank(&sh, 0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (rank != 0 || warp != 0) {
        // helpers: wait for a node to prepare until the walker says it is done
        while (true) {
            cluster.sync();  // A
            const int nd = ctl->cmd;
            if (nd < 0) break;
            prepare_node(sh, ctl, rank, x, n, nd, vec != 0);
            cluster.sync();  // B
        }
        cluster.sync();  // nobody leaves while CTA 0's shared memory may still be read
        return;
    }

    float s = 0.0f;
    int node_opens = 0, tile_opens = 0, leaf_opens = 0;
    WalkClock clk = {0, 0, 0, 0, 0, 0};
    const long long t_begin = walk_clock();
    for (int g0 = 0; g0 < nnodes; g0 += 32) {
        const int count = min(32, nnodes - g0);
        const int node = g0 + lane;
        int2 h = make_int2(0, 0);
        Summ na = summ_invalid(), nb = summ_invalid();
        if (lane < count) {
            h = hyp[node];
            const int4 a = nodeA[node], b = nodeB[node];
            na = {a.x, a.y, a.z, a.w};
            nb = {b.x, b.y, b.z, b.w};
        }
        // both hypotheses of a group's nodes may differ from node to node; the level works with two
        // binades, so take those of the group's first node and let other nodes report "invalid"
        const int gE0 = __shfl_sync(0xffffffffu, h.x, 0), gE1 = __shfl_sync(0xffffffffu, h.y, 0);
        auto node_summ = [&](int E) {
            if (E == h.x) return na;
            if (E == h.y) return nb;
            return summ_invalid();
        };
        s = walk_level(
            s, count, gE0, gE1, [&](int k) { return node_summ(k ? gE1 : gE0); },
            [&](int E) { return node_summ(E); },
            [&](int j, float sj) {
                // open node g0 + j: the cluster prepares its tiles under the exact binade of the
                // state and the neighbouring binade the state is closer to
                if (lane == 0) {
                    const int E = exp_field(sj);
                    sh.e[0] = E;
                    sh.e[1] = (__float_as_int(sj) & 0x400000) ? E + 1 : E - 1;
                    sh.cmd = g0 + j;
                }
                const long long tp = walk_clock();
                cluster.sync();  // A
                prepare_node(sh, ctl, 0, x, n, g0 + j, vec != 0);
                cluster.sync();  // B
                clk.prepare += walk_clock() - tp;
                const int e0 = sh.e[0], e1 = sh.e[1];
                const WalkShared *mine = cluster.map_shared_rank(&sh, lane / TPC);  // holds tile `lane`
                const Summ ta = mine->tile[0][lane % TPC], tb = mine->tile[1][lane % TPC];
                return walk_level(
                    sj, 32, e0, e1, [&](int k) { return k ? tb : ta; },
                    [&](int) { return summ_invalid(); },
                    [&](int jt, float st) {
                        // open tile jt: its 32 leaves, summarised under the same two binades
                        const long long tl0 = walk_clock();
                        const WalkShared *own = cluster.map_shared_rank(&sh, jt / TPC);
                        const int jl = jt % TPC;
                        float v[LEAF];
                        const float4 *src = reinterpret_cast<const float4 *>(&own->raw[jl][lane * RUN_PITCH]);
#pragma unroll
                        for (int i = 0; i < LEAF / 4; i++) {
                            float4 t = src[i];
                            v[4 * i] = t.x, v[4 * i + 1] = t.y, v[4 * i + 2] = t.z, v[4 * i + 3] = t.w;
                        }
                        LeafCtx ca, cb;
                        ca.lo = own->leaf_lo[0][jl][lane], ca.hi = own->leaf_hi[0][jl][lane];
                        ca.c = own->leaf_c[0][jl][lane], ca.tot = own->leaf_tot[0][jl];
                        ca.invmask = own->leaf_inv[0][jl], ca.E = e0, ca.pos0 = 0;
                        cb.lo = own->leaf_lo[1][jl][lane], cb.hi = own->leaf_hi[1][jl][lane];
                        cb.c = own->leaf_c[1][jl][lane], cb.tot = own->leaf_tot[1][jl];
                        cb.invmask = own->leaf_inv[1][jl], cb.E = e1, cb.pos0 = 0;
                        clk.load += walk_clock() - tl0;
                        return walk_leaves(st, v, ca, cb, leaf_opens, clk);
                    },
                    tile_opens);
            },
            node_opens);
    }
    if (lane == 0) {
        sh.cmd = -1;
        out[0] = __fmul_rn(factor, s);
        // how many nodes / tiles / leaves had to be opened (diagnostics, first 16 bytes of scratch)
        stats[0] = node_opens, stats[1] = tile_opens, stats[2] = leaf_opens, stats[3] = nnodes;
        long long *cl = reinterpret_cast<long long *>(stats + 4);
        cl[0] = walk_clock() - t_begin, cl[1] = clk.prepare, cl[2] = clk.leaf_steps, cl[3] = clk.raw;
        cl[4] = clk.rebuild, cl[5] = clk.load;
    }
    cluster.sync();  // A: releases the helpers
    cluster.sync();  // everybody has read the command
}

// Short chains: one thread walks shared-memory tiles that the rest of the CTA stages.
constexpr int CHAIN_TILE = 4096;
constexpr int CHAIN_THREADS = 256;

__global__ void __launch_bounds__(CHAIN_THREADS)
short_chain_kernel(const float *__restrict__ x, float *__restrict__ out, int64_t n, float factor)
{
    __shared__ __align__(16) float buf[2][CHAIN_TILE];
    const int64_t ntiles = (n + CHAIN_TILE - 1) / CHAIN_TILE;
    const int t = threadIdx.x;
    auto stage = [&](int64_t tile, float *dst) {
        const int64_t e0 = tile * CHAIN_TILE;
        for (int i = t; i < CHAIN_TILE; i += CHAIN_THREADS) dst[i] = (e0 + i < n) ? __ldg(x + e0 + i) : 0.0f;
    };
    float s = 0.0f;
    if (ntiles > 0) stage(0, buf[0]);
    __syncthreads();
    for (int64_t tile = 0; tile < ntiles; tile++) {
        const int cur = (int)(tile & 1);
        if (tile + 1 < ntiles) stage(tile + 1, buf[cur ^ 1]);
        if (t == 0) {
            const float4 *b4 = reinterpret_cast<const float4 *>(buf[cur]);
            // padding is +0.0f, which leaves the chain unchanged
#pragma unroll 4
            for (int i = 0; i < CHAIN_TILE / 4; i++) {
                float4 v = b4[i];
                s = __fadd_rn(s, v.x);
                s = __fadd_rn(s, v.y);
                s = __fadd_rn(s, v.z);
                s = __fadd_rn(s, v.w);
            }
        }
        __syncthreads();
    }
    if (t == 0) out[0] = __fmul_rn(factor, s);
}

constexpr int64_t kShortChain = 1 << 16;  // below this the plain walk is faster than four launches

struct Layout {
    int64_t nnodes;
    size_t off_stats, off_sum, off_hyp, off_nodeA, off_nodeB, total;
};

constexpr size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }

constexpr Layout layout_for(int64_t n)
{
    Layout L{};
    L.nnodes = (n + NODE - 1) / NODE;
    constexpr auto up = up256;
    size_t o = 0;
    L.off_stats = o; o = up(o + 4 * sizeof(int) + 8 * sizeof(long long));
    L.off_sum = o;   o = up(o + (size_t)L.nnodes * sizeof(double));
    L.off_hyp = o;   o = up(o + (size_t)L.nnodes * sizeof(int2));
    L.off_nodeA = o; o = up(o + (size_t)L.nnodes * sizeof(int4));
    L.off_nodeB = o; o = up(o + (size_t)L.nnodes * sizeof(int4));
    L.total = o;
    return L;
}

}  // namespace

int sum1d_plain(const float *x, float *out, int64_t n, float factor, cudaStream_t st)
{
    short_chain_kernel<<<1, CHAIN_THREADS, 0, st>>>(x, out, n, factor);
    return launch_status();
}

}  // namespace repdl_b200

using namespace repdl_b200;

extern "C" size_t repdl_b200_sum1d_scratch_bytes(int64_t n)
{
    if (n < kShortChain) return 0;
    return layout_for(n).total;
}

// The four launches of a long chain on scratch memory `base` (device address, 256-byte aligned,
// at least layout_for(n).total bytes).  Nothing in the scratch has to be initialised: every word
// that is read has been written earlier in the same call.
static int sum1d_long(const float *x, float *out, int64_t n, float factor, char *base, cudaStream_t st)
{
    const Layout L = layout_for(n);
    if (L.nnodes > 0x7FFFFFFF / 32) return REPDL_E_RANGE;
    double *node_sum = reinterpret_cast<double *>(base + L.off_sum);
    int2 *hyp = reinterpret_cast<int2 *>(base + L.off_hyp);
    int4 *nodeA = reinterpret_cast<int4 *>(base + L.off_nodeA);
    int4 *nodeB = reinterpret_cast<int4 *>(base + L.off_nodeB);
    const int vec = aligned16(x) ? 1 : 0;
    const unsigned nn = (unsigned)L.nnodes;
    int e;
    node_sum_kernel<<<nn, 256, 0, st>>>(x, n, node_sum, vec);
    if ((e = launch_status())) return e;
    node_scan_kernel<<<1, 1024, 0, st>>>(node_sum, (int)nn, hyp);
    if ((e = launch_status())) return e;
    summarise_kernel<<<nn, 256, 0, st>>>(x, n, hyp, nodeA, nodeB, vec);
    if ((e = launch_status())) return e;
    static unsigned long long smem_done = 0;
    if ((e = ensure_smem(walk_kernel, WALK_SMEM_BYTES, &smem_done))) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(WALK_CLUSTER);
    cfg.blockDim = dim3(WALK_THREADS);
    cfg.dynamicSmemBytes = WALK_SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = WALK_CLUSTER;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, walk_kernel, x, n, (int)nn, (const int2 *)hyp,
                                        (const int4 *)nodeA, (const int4 *)nodeB, factor, out, vec,
                                        reinterpret_cast<int *>(base + L.off_stats));
    if (le != cudaSuccess) {
        (void)cudaGetLastError();
        return (int)le;
    }
    return launch_status();
}

extern "C" int repdl_b200_sum1d(const float *x, float *out, int64_t n, float factor, void *scratch,
                                size_t scratch_bytes, void *stream)
{
    clear_stale_error();
    if (n < 0) return REPDL_E_SHAPE;
    if (!out || (n > 0 && !x)) return REPDL_E_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    if (n < kShortChain) return sum1d_plain(x, out, n, factor, st);
    if (!scratch || scratch_bytes < layout_for(n).total ||
        (reinterpret_cast<uintptr_t>(scratch) & 255u))
        return REPDL_E_SCRATCH;
    return sum1d_long(x, out, n, factor, static_cast<char *>(scratch), st);
}

// ------------------------------------------------------------------------------------------------
// The same chain sum for callers that must not allocate: the scratch is a fixed array in this
// library's device image instead of a buffer the caller provides.
// ------------------------------------------------------------------------------------------------
namespace {
constexpr int64_t kStaticMaxN = (int64_t)1 << 30;                    // 2^30 elements (4 GiB of input)
constexpr size_t kStaticScratchBytes = layout_for(kStaticMaxN).total;  // about 1.5 MB
constexpr int kMaxDevices = 64;
}  // namespace

// Lives in the device image of every GPU that loads this library, for the life of the process.
static __device__ __align__(256) unsigned char g_sum1d_static_scratch[kStaticScratchBytes];

// In host code `g_sum1d_static_scratch` is only a handle for the symbol, not something a kernel can
// dereference; the address the kernels need is asked for once per device, with that device current.
static void *g_static_scratch_addr[kMaxDevices];

extern "C" int64_t repdl_b200_sum1d_static_max_n(void) { return kStaticMaxN; }

extern "C" int repdl_b200_sum1d_static(const float *x, float *out, int64_t n, float factor,
                                       void *stream)
{
    clear_stale_error();
    if (n < 0) return REPDL_E_SHAPE;
    if (n > kStaticMaxN) return REPDL_E_STATIC_MAX;  // the built-in scratch is sized for kStaticMaxN elements
    if (!out || (n > 0 && !x)) return REPDL_E_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    if (n < kShortChain) return sum1d_plain(x, out, n, factor, st);
    int dev = 0;
    cudaError_t ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess) return (int)ce;
    if (dev < 0 || dev >= kMaxDevices) return REPDL_E_RANGE;
    void *addr = __atomic_load_n(&g_static_scratch_addr[dev], __ATOMIC_ACQUIRE);
    if (!addr) {
        // first call on this device: resolve the symbol's device address (no allocation happens;
        // two threads racing here obtain the same address)
        ce = cudaGetSymbolAddress(&addr, g_sum1d_static_scratch);
        if (ce != cudaSuccess) return (int)ce;
        if (!addr) return REPDL_E_SCRATCH;
        __atomic_store_n(&g_static_scratch_addr[dev], addr, __ATOMIC_RELEASE);
    }
    // nothing in the scratch needs clearing: each call writes every word before reading it
    return sum1d_long(x, out, n, factor, static_cast<char *>(addr), st);
}
