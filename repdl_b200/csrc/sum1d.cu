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
// grid is finer) and no state reaches 2^24: m + lo >= 2^23 and m + hi < 2^24, with lo the minimum
// over the steps of (increment so far + floor(q)) and hi the maximum prefix increment.  Such
// summaries (D0, D1, lo, hi) compose associatively, so they can be built by a tree in parallel.
// (For s < 0 the same summary applies to |m| with all four numbers negated and lo/hi swapped.)
//
// Pipeline (all deterministic, no atomics):
//   1. node_sum_kernel      fp64 sum of every node of 32768 elements (only used to PREDICT)
//   2. node_scan_kernel     exclusive scan of those sums -> predicted chain state at each node
//                           start, and from it two binade hypotheses per node: the predicted
//                           binade and its nearer neighbour
//   3. summarise_kernel     per node: leaf summaries (32 elements per lane) under both hypotheses,
//                           composed to one summary per tile of 1024 elements and per node
//   4. walk_kernel          ONE warp carries the exact fp32 state through the nodes: 32 node
//                           summaries are composed by a warp scan and applied in one step when
//                           they are valid for the exact state; the first node that is not valid
//                           (a real binade change, a wrong prediction, a huge element, inf/NaN) is
//                           opened: its 32 tiles are handled the same way, an invalid tile is
//                           loaded and its 32 leaves are summarised on the fly under the exact
//                           binade, and an invalid leaf is finally walked with 32 real fp32 adds.
// A wrong prediction therefore costs time, never bits: every summary is applied only after its
// validity has been checked against the exact state, and everything else is real fp32 addition.
// Elements past n are treated as +0.0f, which never changes a chain that started at +0 (such a
// chain cannot hold -0).
#include "common.cuh"

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

__device__ __forceinline__ Summ summ_negate(const Summ &s)
{
    if (summ_is_invalid(s)) return s;
    return {-s.d0, -s.d1, s.hi <= -BIGI / 2 ? BIGI : -s.hi, s.lo >= BIGI / 2 ? -BIGI : -s.lo};
}

__device__ __forceinline__ Summ shfl_summ(const Summ &s, int src)
{
    return {__shfl_sync(0xffffffffu, s.d0, src), __shfl_sync(0xffffffffu, s.d1, src),
            __shfl_sync(0xffffffffu, s.lo, src), __shfl_sync(0xffffffffu, s.hi, src)};
}

__device__ __forceinline__ Summ shfl_up_summ(const Summ &s, int delta)
{
    return {__shfl_up_sync(0xffffffffu, s.d0, delta), __shfl_up_sync(0xffffffffu, s.d1, delta),
            __shfl_up_sync(0xffffffffu, s.lo, delta), __shfl_up_sync(0xffffffffu, s.hi, delta)};
}

// Summary of the elements v[0..LEAF) (in order) under binade hypothesis E (exponent field).
// Hypotheses outside [24, 253] are not summarised (the scale 2^(150-E) must be a finite float).
__device__ __forceinline__ Summ leaf_summary(const float (&v)[LEAF], int E)
{
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
        // The step is modelled correctly iff its exact value m + q is not below 2^23, i.e. iff
        // m + D_before + floor(q) >= 2^23 (m and D are integers); floor(q) = R - (d < 0).
        lo = min(lo, d0 + R + (__float_as_int(d) >> 31));
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
        hi = max(hi, d0);
    }
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

// One level of the walk.  `count` children (<= 32), child c owned by lane c.
//   get(E, negative) -> this lane's summary for a state in binade E (already negated for s < 0),
//                       or an invalid summary;
//   open(j, s)       -> the exact state after child j entered with state s (uniform call).
// Returns the exact state after all children.
template <class Get, class Open>
__device__ __forceinline__ float walk_level(float s, int count, Get get, Open open, int &opens)
{
    const int lane = threadIdx.x & 31;
    int pos = 0;
    while (pos < count) {
        const int E = exp_field(s);
        const bool neg = __float_as_int(s) < 0;
        Summ mine = (lane >= pos && lane < count) ? get(E, neg) : summ_identity();
        if (E < 24 || E > 253) mine = (lane >= pos && lane < count) ? summ_invalid() : summ_identity();
        // inclusive scan of composition over the lanes
        Summ incl = mine;
#pragma unroll
        for (int dlt = 1; dlt < 32; dlt <<= 1) {
            Summ up = shfl_up_summ(incl, dlt);
            if (lane >= dlt) incl = summ_compose(up, incl);
        }
        Summ excl = shfl_up_summ(incl, 1);
        if (lane == 0) excl = summ_identity();
        const int m = (int)(((unsigned)__float_as_int(s) & 0x7FFFFFu) | 0x800000u);
        const int par = m & 1;
        bool ok = true;
        if (lane >= pos && lane < count) {
            if (summ_is_invalid(excl) || summ_is_invalid(mine)) {
                ok = false;
            } else {
                const int m_in = m + (par ? excl.d1 : excl.d0);
                ok = (m_in + mine.lo >= M_LO) && (m_in + mine.hi < M_HI);
            }
        }
        const unsigned badmask = __ballot_sync(0xffffffffu, !ok);
        if (badmask == 0u) {
            const Summ tot = shfl_summ(incl, 31);
            return apply_inc(s, par ? tot.d1 : tot.d0);
        }
        const int j = __ffs((int)badmask) - 1;
        const Summ before = shfl_summ(excl, j);  // valid: every lane in [pos, j) checked ok
        if (j > pos) s = apply_inc(s, par ? before.d1 : before.d0);
        s = open(j, s);
        opens++;
        pos = j + 1;
    }
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
// 3. summaries of tiles and nodes under both hypotheses
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
                 int4 *__restrict__ tileA, int4 *__restrict__ tileB, int4 *__restrict__ nodeA,
                 int4 *__restrict__ nodeB, int vec)
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
            tileA[(int64_t)node * 32 + tl] = make_int4(a.d0, a.d1, a.lo, a.hi);
            tileB[(int64_t)node * 32 + tl] = make_int4(b.d0, b.d1, b.lo, b.hi);
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
// 4. the walk (one warp)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ Summ pick(int E, bool neg, int2 h, int4 a, int4 b)
{
    Summ s;
    if (E == h.x)
        s = {a.x, a.y, a.z, a.w};
    else if (E == h.y)
        s = {b.x, b.y, b.z, b.w};
    else
        return summ_invalid();
    return neg ? summ_negate(s) : s;
}

__global__ void __launch_bounds__(32)
walk_kernel(const float *__restrict__ x, int64_t n, int nnodes, const int2 *__restrict__ hyp,
            const int4 *__restrict__ tileA, const int4 *__restrict__ tileB,
            const int4 *__restrict__ nodeA, const int4 *__restrict__ nodeB, float factor,
            float *__restrict__ out, int vec, int *__restrict__ stats)
{
    const int lane = threadIdx.x;
    float s = 0.0f;
    int node_opens = 0, tile_opens = 0, leaf_opens = 0;
    for (int g0 = 0; g0 < nnodes; g0 += 32) {
        const int count = min(32, nnodes - g0);
        const int node = g0 + lane;
        int2 h = make_int2(0, 0);
        int4 na = make_int4(0, 0, 0, 0), nb = na;
        if (lane < count) {
            h = hyp[node];
            na = nodeA[node];
            nb = nodeB[node];
        }
        s = walk_level(
            s, count, [&](int E, bool neg) { return pick(E, neg, h, na, nb); },
            [&](int j, float sj) {
                // open node g0 + j: its 32 tiles
                const int nd = g0 + j;
                const int2 hn = hyp[nd];
                const int4 ta = tileA[(int64_t)nd * 32 + lane], tb = tileB[(int64_t)nd * 32 + lane];
                return walk_level(
                    sj, 32, [&](int E, bool neg) { return pick(E, neg, hn, ta, tb); },
                    [&](int jt, float st) {
                        // open tile jt of the node: 32 leaves, summarised under the exact binade
                        float v[LEAF];
                        load_leaf(x, n, (int64_t)nd * NODE + (int64_t)jt * TILE, vec != 0, v);
                        return walk_level(
                            st, 32,
                            [&](int E, bool neg) {
                                Summ q = leaf_summary(v, E);
                                return neg ? summ_negate(q) : q;
                            },
                            [&](int jl, float sl) {
                                // open leaf jl: 32 real fp32 adds by its owner
                                float r = sl;
                                if (lane == jl) {
#pragma unroll
                                    for (int i = 0; i < LEAF; i++) r = __fadd_rn(r, v[i]);
                                }
                                return __shfl_sync(0xffffffffu, r, jl);
                            },
                            leaf_opens);
                    },
                    tile_opens);
            },
            node_opens);
    }
    if (lane == 0) {
        out[0] = __fmul_rn(factor, s);
        // how many nodes / tiles / leaves had to be opened (diagnostics, first 16 bytes of scratch)
        stats[0] = node_opens, stats[1] = tile_opens, stats[2] = leaf_opens, stats[3] = nnodes;
    }
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
    size_t off_stats, off_sum, off_hyp, off_nodeA, off_nodeB, off_tileA, off_tileB, total;
};

Layout layout_for(int64_t n)
{
    Layout L;
    L.nnodes = (n + NODE - 1) / NODE;
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    size_t o = 0;
    L.off_stats = o; o = up(o + 4 * sizeof(int));
    L.off_sum = o;   o = up(o + (size_t)L.nnodes * sizeof(double));
    L.off_hyp = o;   o = up(o + (size_t)L.nnodes * sizeof(int2));
    L.off_nodeA = o; o = up(o + (size_t)L.nnodes * sizeof(int4));
    L.off_nodeB = o; o = up(o + (size_t)L.nnodes * sizeof(int4));
    L.off_tileA = o; o = up(o + (size_t)L.nnodes * 32 * sizeof(int4));
    L.off_tileB = o; o = up(o + (size_t)L.nnodes * 32 * sizeof(int4));
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

extern "C" int repdl_b200_sum1d(const float *x, float *out, int64_t n, float factor, void *scratch,
                                size_t scratch_bytes, void *stream)
{
    clear_stale_error();
    if (n < 0) return REPDL_E_SHAPE;
    if (!out || (n > 0 && !x)) return REPDL_E_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    if (n < kShortChain) return sum1d_plain(x, out, n, factor, st);
    const Layout L = layout_for(n);
    if (L.nnodes > 0x7FFFFFFF / 32) return REPDL_E_RANGE;
    if (!scratch || scratch_bytes < L.total || (reinterpret_cast<uintptr_t>(scratch) & 255u))
        return REPDL_E_SCRATCH;
    char *base = static_cast<char *>(scratch);
    double *node_sum = reinterpret_cast<double *>(base + L.off_sum);
    int2 *hyp = reinterpret_cast<int2 *>(base + L.off_hyp);
    int4 *nodeA = reinterpret_cast<int4 *>(base + L.off_nodeA);
    int4 *nodeB = reinterpret_cast<int4 *>(base + L.off_nodeB);
    int4 *tileA = reinterpret_cast<int4 *>(base + L.off_tileA);
    int4 *tileB = reinterpret_cast<int4 *>(base + L.off_tileB);
    const int vec = aligned16(x) ? 1 : 0;
    const unsigned nn = (unsigned)L.nnodes;
    int e;
    node_sum_kernel<<<nn, 256, 0, st>>>(x, n, node_sum, vec);
    if ((e = launch_status())) return e;
    node_scan_kernel<<<1, 1024, 0, st>>>(node_sum, (int)nn, hyp);
    if ((e = launch_status())) return e;
    summarise_kernel<<<nn, 256, 0, st>>>(x, n, hyp, tileA, tileB, nodeA, nodeB, vec);
    if ((e = launch_status())) return e;
    walk_kernel<<<1, 32, 0, st>>>(x, n, (int)nn, hyp, tileA, tileB, nodeA, nodeB, factor, out, vec,
                                  reinterpret_cast<int *>(base + L.off_stats));
    return launch_status();
}
