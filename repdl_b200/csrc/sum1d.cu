// sum1d: ONE strict left-to-right fp32 chain over n elements (microsoft/RepDL
// backend/cpu/summation.cpp:12-20: `sum += I[i]` from +0, then `factor * sum`), reproduced bit for
// bit but not walked element by element.
//
// The algebra (per-binade integer summaries of runs of elements, their validity condition and
// composition) is in sum1d_core.cuh.  The exact chain state is a serial dependency, so the pipeline
// does in parallel everything that does NOT need it and leaves one thread a short list of things
// that do:
//   1. tile_sum_kernel   fp64 sums of every tile (1024 elements) and node (32768 elements)
//   2. predict_kernel    exclusive scan of the node sums -> the PREDICTED chain state at each node
//                        start, and a bound on how far the fp32 chain may have drifted from the
//                        prediction by then (random-walk model of the roundings, 5 sigma)
//   3. classify_kernel   per node: every leaf (32 elements) is summarised under the binade its
//                        predicted entry state lies in and classified: robust (valid for every
//                        state within the drift bound), soft (valid for the prediction itself) or
//                        hard.  A node whose leaves are all robust under one binade becomes a
//                        single summary; any other node reports how many items it needs.
//   4. plan_kernel       exclusive scan of the item counts -> where each node's items go
//   5. emit_kernel       writes the item stream: runs of robust leaves composed into one item,
//                        runs of soft leaves as one composed item followed by its leaves (so that a
//                        valid run is one step and an invalid one falls through to its leaves),
//                        hard leaves as "walk these 32 elements"
//   6. walk_kernel       one CTA: thread 0 carries the exact fp32 state through the items -- a
//                        summary is applied only after its validity has been checked against the
//                        exact state, everything else is real fp32 addition -- while the other
//                        warps stage the next batch of items and the elements of its leaves in
//                        shared memory.
// A wrong prediction therefore costs time, never bits.  Elements past n are treated as +0.0f, which
// never changes a chain that started at +0 (such a chain cannot hold -0).
#include "common.cuh"
#include "sum1d_core.cuh"
#include "sum1d_walk.cuh"

namespace repdl_b200 {
namespace {

using namespace s1;

enum NodeKind { N_SMOOTH = 0, N_MIXED = 1, N_RAW = 2 };

struct __align__(16) NodeRec {
    Summ pos;         // composed positive-orientation summary (N_SMOOTH)
    int sek;          // its hypothesis
    int kind, count;  // NodeKind; items this node contributes
    int off;          // index of its first item (plan_kernel)
};
static_assert(sizeof(NodeRec) == 32, "two 16-byte words");

struct Header {
    int total_items;  // plan_kernel
    int error;        // emit_kernel: a node produced a different item count than it announced
    int pad[2];
    long long stats[12];  // walk_kernel: see repdl_b200_sum1d_stats
};

__device__ __forceinline__ double shfl_up_d(double v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }
__device__ __forceinline__ double shfl_down_d(double v, int d) { return __shfl_down_sync(0xffffffffu, v, d); }

// ---------------------------------------------------------------------------------------------
// 1. fp64 sum per tile and per node (prediction only)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
tile_sum_kernel(const float *__restrict__ x, int64_t n, double *__restrict__ tile_sum,
                double *__restrict__ node_sum, int vec)
{
    __shared__ double ts[TILES_PER_NODE];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t node = blockIdx.x;
#pragma unroll 1
    for (int t = warp; t < TILES_PER_NODE; t += 8) {
        const int64_t base = node * NODE + (int64_t)t * TILE;
        double acc = 0.0;
        if (vec && base + TILE <= n) {
            const float4 *p = reinterpret_cast<const float4 *>(x + base);
            float4 v[8];
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = __ldg(p + j * 32 + lane);
#pragma unroll
            for (int j = 0; j < 8; j++)
                acc += ((double)v[j].x + (double)v[j].y) + ((double)v[j].z + (double)v[j].w);
        } else {
            for (int i = lane; i < TILE; i += 32)
                if (base + i < n) acc += (double)__ldg(x + base + i);
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) acc += shfl_down_d(acc, d);
        if (lane == 0) {
            ts[t] = acc;
            tile_sum[node * TILES_PER_NODE + t] = acc;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        double s = 0.0;
        for (int t = 0; t < TILES_PER_NODE; t++) s += ts[t];
        node_sum[node] = s;
    }
}

// ---------------------------------------------------------------------------------------------
// 2. predicted state and drift bound at every node start (one CTA)
// ---------------------------------------------------------------------------------------------
// Exclusive scan of one value per thread over the 1024 threads of the CTA.
__device__ __forceinline__ double block_exclusive_scan_1024(double v, double *wtot)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    double incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const double up = shfl_up_d(incl, d);
        if (lane >= d) incl += up;
    }
    __syncthreads();  // wtot may still be read from an earlier scan
    if (lane == 31) wtot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const double w = wtot[lane];
        double wi = w;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const double up = shfl_up_d(wi, d);
            if (lane >= d) wi += up;
        }
        wtot[lane] = wi - w;
    }
    __syncthreads();
    return wtot[warp] + (incl - v);
}

__global__ void __launch_bounds__(1024)
predict_kernel(const double *__restrict__ node_sum, int nnodes, double *__restrict__ pred,
               double *__restrict__ rabs)
{
    // Thread t owns the consecutive nodes [t * per, (t + 1) * per) of every slab of 1024 * per
    // nodes; a slab goes through shared memory so that global memory is read and written in order.
    constexpr int PER = 4;
    __shared__ double wtot[32];
    __shared__ double slab[1024 * PER + 1024 * PER / 32];  // padded: thread-consecutive reads without conflicts
    __shared__ double carry_run, carry_var;
    const int t = threadIdx.x;
    if (t == 0) carry_run = 0.0, carry_var = 0.0;
    __syncthreads();
    auto at = [](int i) { return i + (i >> 5); };
    for (int base = 0; base < nnodes; base += 1024 * PER) {
        const int count = min(1024 * PER, nnodes - base);
        for (int i = t; i < 1024 * PER; i += 1024) slab[at(i)] = i < count ? node_sum[base + i] : 0.0;
        __syncthreads();
        double v[PER], s = 0.0;
#pragma unroll
        for (int k = 0; k < PER; k++) v[k] = slab[at(t * PER + k)], s += v[k];
        double run = carry_run + block_exclusive_scan_1024(s, wtot);
        double dv[PER], vs = 0.0;
#pragma unroll
        for (int k = 0; k < PER; k++) {
            const double a = fabs(run);
            slab[at(t * PER + k)] = run;  // predicted state at the node's start
            run += v[k];
            dv[k] = drift_variance(fmax(a, fabs(run)));
            vs += dv[k];
        }
        __syncthreads();
        for (int i = t; i < count; i += 1024) pred[base + i] = slab[at(i)];
        double var = carry_var + block_exclusive_scan_1024(vs, wtot);  // (syncs: the slab is free again)
#pragma unroll
        for (int k = 0; k < PER; k++) {
            var += dv[k];
            slab[at(t * PER + k)] = DRIFT_SIGMAS * sqrt(var);
        }
        __syncthreads();
        for (int i = t; i < count; i += 1024) rabs[base + i] = slab[at(i)];
        if (t == 1023) carry_run = run, carry_var = var;
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// 3./5. leaf classification of one node (shared by classify_kernel and emit_kernel)
// ---------------------------------------------------------------------------------------------
constexpr int RUN_PITCH = 36;  // floats per lane-run in shared memory: LDS.128 without bank conflicts

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

// Loads tile [base, base + TILE) so that lane l ends up with its leaf [base + 32 l, +32) in v:
// coalesced 16-byte loads, transposed through the warp's private shared-memory buffer.
__device__ __forceinline__ void load_tile_leaves(const float *__restrict__ x, int64_t n, int64_t base,
                                                 bool vec, float *tbuf, float (&v)[LEAF])
{
    const int lane = threadIdx.x & 31;
    if (vec && base + TILE <= n) {
        const float4 *p = reinterpret_cast<const float4 *>(x + base);
        float4 t[8];
#pragma unroll
        for (int j = 0; j < 8; j++) t[j] = __ldg(p + j * 32 + lane);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int idx = j * 32 + lane;  // float4 index in the tile: leaf idx / 8, quad idx % 8
            *reinterpret_cast<float4 *>(&tbuf[(idx >> 3) * RUN_PITCH + (idx & 7) * 4]) = t[j];
        }
    } else {
        for (int i = lane; i < TILE; i += 32)
            tbuf[(i >> 5) * RUN_PITCH + (i & 31)] = (base + i < n) ? __ldg(x + base + i) : 0.0f;
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < LEAF / 4; i++) {
        const float4 q = *reinterpret_cast<const float4 *>(&tbuf[lane * RUN_PITCH + 4 * i]);
        v[4 * i] = q.x, v[4 * i + 1] = q.y, v[4 * i + 2] = q.z, v[4 * i + 3] = q.w;
    }
    __syncwarp();
}

// Classifies the 1024 leaves of `node`: code[] (class and hypothesis per leaf) and, if KEEP, the
// positive-orientation summary of every leaf in summ[]; otherwise the composed summary of every
// tile in tile_summ[].  NW warps; tbuf holds NW * 32 * RUN_PITCH floats; tpre 32 doubles.
template <int NW, bool KEEP>
__device__ __forceinline__ void classify_node_leaves(const float *__restrict__ x, int64_t n, int64_t node,
                                                     bool vec, const double *__restrict__ tile_sum,
                                                     double pred, double rabs, float *tbuf, double *tpre,
                                                     unsigned short *code, Summ *summ, Summ *tile_summ)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) {
        const double ts = tile_sum[node * TILES_PER_NODE + lane];
        double incl = ts;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const double up = shfl_up_d(incl, d);
            if (lane >= d) incl += up;
        }
        tpre[lane] = pred + (incl - ts);
    }
    __syncthreads();
    float *my = tbuf + warp * 32 * RUN_PITCH;
#pragma unroll 1
    for (int t = warp; t < TILES_PER_NODE; t += NW) {
        float v[LEAF];
        load_tile_leaves(x, n, node * NODE + (int64_t)t * TILE, vec, my, v);
        // the leaf's sum, for the prediction only: an fp32 tree (its error is far below the drift
        // bound; fp64 conversions and additions per element would cost half as much as the summary)
        float t8[8];
#pragma unroll
        for (int i = 0; i < 8; i++)
            t8[i] = __fadd_rn(__fadd_rn(v[4 * i], v[4 * i + 1]), __fadd_rn(v[4 * i + 2], v[4 * i + 3]));
        const double ls = (double)__fadd_rn(__fadd_rn(__fadd_rn(t8[0], t8[1]), __fadd_rn(t8[2], t8[3])),
                                            __fadd_rn(__fadd_rn(t8[4], t8[5]), __fadd_rn(t8[6], t8[7])));
        double incl = ls;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const double up = shfl_up_d(incl, d);
            if (lane >= d) incl += up;
        }
        const double p = tpre[t] + (incl - ls);
        const int sek = hyp_sign_exp(p);
        const Summ sm = leaf_summary(v, sek & 255);
        const int cls = classify_leaf(sm, sek, p, rabs);
        code[t * 32 + lane] = (unsigned short)leaf_code(cls, sek);
        if (KEEP) {
            summ[t * 32 + lane] = sm;
        } else {
            const Summ ts = warp_reduce_summ(sm);
            if (lane == 0) tile_summ[t] = ts;
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(256)
classify_kernel(const float *__restrict__ x, int64_t n, const double *__restrict__ tile_sum,
                const double *__restrict__ pred, const double *__restrict__ rabs,
                NodeRec *__restrict__ rec, int vec)
{
    __shared__ __align__(16) float tbuf[8 * 32 * RUN_PITCH];
    __shared__ double tpre[TILES_PER_NODE];
    __shared__ unsigned short code[LEAVES_PER_NODE];
    __shared__ Summ tile_summ[TILES_PER_NODE];
    __shared__ int wcount[8], wsmooth[8];
    const int64_t node = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    classify_node_leaves<8, false>(x, n, node, vec != 0, tile_sum, pred[node], rabs[node], tbuf, tpre, code,
                                   nullptr, tile_summ);
    int count = 0;
    bool smooth = true;
    const int c0 = code[0];
    for (int i = threadIdx.x; i < LEAVES_PER_NODE; i += 256) {
        count += leaf_item_count(code, i);
        smooth &= code[i] == c0;
    }
    smooth &= code_class(c0) == C_ROBUST;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) count += __shfl_down_sync(0xffffffffu, count, d);
    const bool wsm = __all_sync(0xffffffffu, smooth);
    if (lane == 0) wcount[warp] = count, wsmooth[warp] = wsm;
    __syncthreads();
    if (warp == 0) {
        const Summ acc = warp_reduce_summ(tile_summ[lane]);
        if (lane == 0) {
            int total = 0;
            bool sm = true;
            for (int w = 0; w < 8; w++) total += wcount[w], sm &= wsmooth[w] != 0;
            NodeRec r;
            if (sm)
                r = {acc, code_sek(c0), N_SMOOTH, 1, 0};
            else
                r = {summ_invalid(), 0, N_MIXED, total, 0};
            rec[node] = r;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// 4. where each node's items go (one CTA).  From the first node whose items would no longer fit
// into the buffer (one slot is kept for each later node), every node becomes one raw span.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ long long block_exclusive_scan_ll_1024(long long v, long long *wtot)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    long long incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const long long up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
    }
    __syncthreads();
    if (lane == 31) wtot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const long long w = wtot[lane];
        long long wi = w;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const long long up = __shfl_up_sync(0xffffffffu, wi, d);
            if (lane >= d) wi += up;
        }
        wtot[lane] = wi - w;
    }
    __syncthreads();
    return wtot[warp] + (incl - v);
}

// Consecutive smooth nodes under one hypothesis are merged: a header item (kind K_SOFT: applied ->
// the nodes' own items are skipped, not valid -> the walker goes on to them) carries their composed
// summary.  A merged stretch never crosses the boundary between two threads' chunks of nodes, so
// each thread plans its chunk alone.
template <bool WRITE>
__device__ __forceinline__ long long plan_chunk(NodeRec *__restrict__ rec, int lo, int hi, long long run,
                                                Item *__restrict__ items)
{
    int i = lo;
    while (i < hi) {
        const NodeRec r = rec[i];
        if (r.kind != N_SMOOTH) {
            if (WRITE) rec[i].off = (int)run;
            run += r.count;
            i++;
            continue;
        }
        int j = i + 1;
        Summ acc = r.pos;
        while (j < hi) {
            const NodeRec q = rec[j];
            if (q.kind != N_SMOOTH || q.sek != r.sek) break;
            if (WRITE) acc = summ_compose(acc, q.pos);
            j++;
        }
        const int len = j - i;
        if (len >= 2) {
            if (WRITE)
                items[run] = make_item(K_SOFT, acc, r.sek, len, i * LEAVES_PER_NODE, len * LEAVES_PER_NODE);
            run++;
        }
        if (WRITE)
            for (int k = i; k < j; k++) rec[k].off = (int)(run + (k - i));
        run += len;
        i = j;
    }
    return run;
}

__global__ void __launch_bounds__(1024)
plan_kernel(NodeRec *__restrict__ rec, int nnodes, long long cap, Header *__restrict__ hdr,
            Item *__restrict__ items)
{
    __shared__ long long wtot[32];
    __shared__ int first_over_sh, wmin[32];
    __shared__ long long over_off_sh, total_sh;
    const int t = threadIdx.x;
    const int per = (nnodes + 1023) / 1024;
    const int lo = min(t * per, nnodes), hi = min(lo + per, nnodes);
    if (t == 0) over_off_sh = 0;
    // with merged stretches, if everything fits
    const long long mine = plan_chunk<false>(rec, lo, hi, 0, nullptr);
    const long long mbase = block_exclusive_scan_ll_1024(mine, wtot);
    if (t == 1023) total_sh = mbase + mine;
    __syncthreads();
    if (total_sh <= cap) {
        plan_chunk<true>(rec, lo, hi, mbase, items);
        if (t == 1023) {
            hdr->total_items = (int)total_sh;
            hdr->error = 0;
        }
        return;
    }
    // otherwise no merging, and from the first node whose items would no longer fit (one slot is
    // kept for each later node) every node becomes one raw span
    long long s = 0;
    for (int i = lo; i < hi; i++) s += rec[i].count;
    const long long base = block_exclusive_scan_ll_1024(s, wtot);
    long long run = base;
    int my_over = nnodes;
    for (int i = lo; i < hi; i++) {
        const int c = rec[i].count;
        if (my_over == nnodes && run + c + (long long)(nnodes - i - 1) > cap) my_over = i;
        run += c;
    }
    // block minimum of my_over (shuffles, then one pass over the 32 warp minima)
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) my_over = min(my_over, __shfl_xor_sync(0xffffffffu, my_over, d));
    if ((t & 31) == 0) wmin[t >> 5] = my_over;
    __syncthreads();
    if (t == 0) {
        int m = nnodes;
        for (int w = 0; w < 32; w++) m = min(m, wmin[w]);
        first_over_sh = m;
    }
    __syncthreads();
    const int first_over = first_over_sh;
    run = base;
    for (int i = lo; i < hi; i++) {
        if (i == first_over) over_off_sh = run;
        run += rec[i].count;
    }
    __syncthreads();
    const long long over_off = over_off_sh;
    run = base;
    for (int i = lo; i < hi; i++) {
        const int c = rec[i].count;
        if (i >= first_over) {
            rec[i].kind = N_RAW;
            rec[i].count = 1;
            rec[i].off = (int)(over_off + (i - first_over));
        } else {
            rec[i].off = (int)run;
        }
        run += c;
    }
    if (t == 1023) {
        hdr->total_items = first_over < nnodes ? (int)(over_off + (nnodes - first_over)) : (int)run;
        hdr->error = 0;
    }
}

// ---------------------------------------------------------------------------------------------
// 5. the item stream
// ---------------------------------------------------------------------------------------------
constexpr int EMIT_WARPS = 4;

__global__ void __launch_bounds__(EMIT_WARPS * 32)
emit_kernel(const float *__restrict__ x, int64_t n, const double *__restrict__ tile_sum,
            const double *__restrict__ pred, const double *__restrict__ rabs,
            const NodeRec *__restrict__ rec, Item *__restrict__ items, Header *__restrict__ hdr, int vec,
            int64_t nnodes)
{
    __shared__ __align__(16) float tbuf[EMIT_WARPS * 32 * RUN_PITCH];
    __shared__ double tpre[TILES_PER_NODE];
    __shared__ unsigned short code[LEAVES_PER_NODE];
    __shared__ Summ summ[LEAVES_PER_NODE];
    __shared__ int wtot[EMIT_WARPS];
    constexpr int PER = LEAVES_PER_NODE / (EMIT_WARPS * 32);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int64_t node = blockIdx.x; node < nnodes; node += gridDim.x) {
        const NodeRec r = rec[node];
        Item *out = items + r.off;
        const int leaf0 = (int)(node * LEAVES_PER_NODE);
        if (r.kind != N_MIXED) {
            if (threadIdx.x == 0)
                out[0] = r.kind == N_SMOOTH ? make_item(K_RUN, r.pos, r.sek, 0, leaf0, LEAVES_PER_NODE)
                                            : make_item(K_RAWSPAN, summ_invalid(), 0, 0, leaf0, LEAVES_PER_NODE);
            continue;
        }
        classify_node_leaves<EMIT_WARPS, true>(x, n, node, vec != 0, tile_sum, pred[node], rabs[node], tbuf,
                                               tpre, code, summ, nullptr);
        // thread t owns the consecutive leaves [t * PER, (t + 1) * PER)
        const int first = threadIdx.x * PER;
        int mine = 0;
        for (int k = 0; k < PER; k++) mine += leaf_item_count(code, first + k);
        int incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += up;
        }
        if (lane == 31) wtot[warp] = incl;
        __syncthreads();
        int idx = incl - mine;
        for (int w = 0; w < warp; w++) idx += wtot[w];
        for (int k = 0; k < PER; k++) {
            leaf_emit_items(code, summ, first + k, leaf0, out + idx);
            idx += leaf_item_count(code, first + k);
        }
        if (threadIdx.x == EMIT_WARPS * 32 - 1 && idx != r.count) hdr->error = 1;
        __syncthreads();  // the shared arrays are reused by the next node
    }
}

// ---------------------------------------------------------------------------------------------
// Cooperative plain walk of elements [e0, e1): the first warp adds (all its lanes the same values,
// so that the warp never diverges), the other warps stage.  Every thread of the CTA calls it; the
// first warp returns the new state.  buf holds 2 * CHAIN_TILE floats.
// ---------------------------------------------------------------------------------------------
constexpr int CHAIN_TILE = 2048;

__device__ __forceinline__ float coop_chain(const float *__restrict__ x, int64_t e0, int64_t e1, float s,
                                            float *buf)
{
    const int t = threadIdx.x, nt = blockDim.x;
    const int64_t ntiles = e1 > e0 ? (e1 - e0 + CHAIN_TILE - 1) / CHAIN_TILE : 0;
    auto stage = [&](int64_t tile, float *dst, int first, int step) {
        const int64_t b = e0 + tile * CHAIN_TILE;
        for (int i = first; i < CHAIN_TILE; i += step) dst[i] = (b + i < e1) ? __ldg(x + b + i) : 0.0f;
    };
    if (ntiles > 0) stage(0, buf, t, nt);
    __syncthreads();
    for (int64_t tile = 0; tile < ntiles; tile++) {
        float *cur = buf + (tile & 1) * CHAIN_TILE;
        if (t >= 32) {
            if (tile + 1 < ntiles) stage(tile + 1, buf + ((tile + 1) & 1) * CHAIN_TILE, t - 32, nt - 32);
        } else {
            const float4 *b4 = reinterpret_cast<const float4 *>(cur);
            // padding is +0.0f, which leaves the chain unchanged
#pragma unroll 4
            for (int i = 0; i < CHAIN_TILE / 4; i++) {
                const float4 v = b4[i];
                s = __fadd_rn(s, v.x);
                s = __fadd_rn(s, v.y);
                s = __fadd_rn(s, v.z);
                s = __fadd_rn(s, v.w);
            }
        }
        __syncthreads();
    }
    return s;
}

// ---------------------------------------------------------------------------------------------
// 6. the walk
// ---------------------------------------------------------------------------------------------
// Cycle counters of the walker thread (stats[7..12) of the scratch header); compiled out unless asked
// for with -DREPDL_SUM1D_CLOCKS=1, since reading the clock per item is itself part of the walk.
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

constexpr int WALK_THREADS = 256;
#ifndef REPDL_SUM1D_BATCH
#define REPDL_SUM1D_BATCH 256
#endif
constexpr int WALK_BATCH = REPDL_SUM1D_BATCH;  // items per staged batch

struct WalkShared {
    WItem items[2][WALK_BATCH + 1];
    float raw[2][WALK_BATCH][LEAF];  // the elements of a batch's K_LEAF / K_HARD items
    float chain[2 * CHAIN_TILE];
    int cmd[2][4];
};
constexpr int WALK_SMEM_BYTES = (int)sizeof(WalkShared);
enum { CMD_NEXT = 0, CMD_SPAN = 1 };

// Warps 1..7: items [b * WALK_BATCH, +WALK_BATCH) of the stream and the elements of their leaves.
__device__ __forceinline__ void stage_batch(WalkShared &sh, int buf, int b, int total,
                                            const Item *__restrict__ items, const float *__restrict__ x,
                                            int64_t n)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll 1
    for (int r = warp - 1; r < WALK_BATCH / 32; r += WALK_THREADS / 32 - 1) {
        const int slot = r * 32 + lane;
        const int gi = b * WALK_BATCH + slot;
        WItem w = witem_end();  // past the stream: end marker
        if (gi < total) {
            const int4 *src = reinterpret_cast<const int4 *>(items + gi);
            w = witem_from(__ldg(src), __ldg(src + 1));
        }
        const int kind = w.kind;
        sh.items[buf][slot] = w;
        const bool need = gi < total && (kind == K_LEAF || kind == K_HARD);
        const unsigned needmask = __ballot_sync(0xffffffffu, need);
        // the 32 elements of each such leaf: one 4-byte asynchronous copy per lane (zero-filled past
        // n), so that no copy waits for an earlier one
#pragma unroll
        for (int j = 0; j < 32; j++) {
            if ((needmask >> j) & 1u) {
                const int64_t e = (int64_t)__shfl_sync(0xffffffffu, w.start, j) * LEAF + lane;
                cp_async_4_zfill(&sh.raw[buf][r * 32 + j][lane], x + (e < n ? e : 0), e < n);
            }
        }
    }
    if (threadIdx.x == 32) sh.items[buf][WALK_BATCH] = witem_end();
    cp_async_commit();
    cp_async_wait<0>();
}

__global__ void __launch_bounds__(WALK_THREADS, 1)
walk_kernel(const float *__restrict__ x, int64_t n, Header *__restrict__ hdr, const Item *__restrict__ items,
            float factor, float *__restrict__ out)
{
    extern __shared__ __align__(16) unsigned char walk_smem[];
    WalkShared &sh = *reinterpret_cast<WalkShared *>(walk_smem);
    const int tid = threadIdx.x, warp = tid >> 5;
    const int total = hdr->total_items;
    if (hdr->error != 0) {
        // the item stream is not trustworthy: walk the whole chain
        const float s = coop_chain(x, 0, n, 0.0f, sh.chain);
        if (tid == 0) {
            out[0] = __fmul_rn(factor, s);
            hdr->stats[0] = -1;
        }
        return;
    }
    const int nb = (total + WALK_BATCH - 1) / WALK_BATCH;
    if (warp > 0 && nb > 0) stage_batch(sh, 0, 0, total, items, x, n);
    __syncthreads();
    int bits = 0;  // the exact state: +0.0f
    int i = 0;     // next item (thread 0)
    int n_span = 0, n_run_fail = 0;
    WalkCounts counts = {0, 0, 0};
    long long n_span_leaves = 0;
    long long c_items = 0, c_raw = 0, c_span = 0, c_wait = 0, c_pre = 0, c_post = 0;  // walker cycles (diagnostic builds)
    const long long c_begin = walk_clock();
    bool next_staged = false;
    int round = 0;
    for (int bt = 0; bt < nb; round++) {
        const long long c_top = walk_clock();
        const int buf = bt & 1, base = bt * WALK_BATCH, end = min(total, base + WALK_BATCH);
        if (warp == 0) {
            int c = CMD_NEXT;
            const long long c_in = walk_clock();
            c_pre += c_in - c_top;
            const int cnt = end - base;
            int p = (i - base) * (int)sizeof(WItem);
            if (p < cnt * (int)sizeof(WItem)) {
                const long long c_r = walk_clock();
                const int why = walk_batch<REPDL_SUM1D_CLOCKS != 0>(
                    reinterpret_cast<const unsigned char *>(sh.items[buf]), &sh.raw[buf][0][0],
                    cnt * (int)sizeof(WItem), p, bits, counts);
                c_raw += walk_clock() - c_r;
                if (why == WALK_SPAN) {
                    const WItem &it = sh.items[buf][p / (int)sizeof(WItem)];
                    n_run_fail += it.kind == K_RUN;
                    if (tid == 0) {
                        sh.cmd[round & 1][1] = it.start;
                        sh.cmd[round & 1][2] = it.len;
                    }
                    c = CMD_SPAN;
                }
            }
            const int idx = p / (int)sizeof(WItem);
            i = base + idx;
            if (tid == 0) sh.cmd[round & 1][0] = c;
            c_items += walk_clock() - c_in;
        } else if (warp > 0 && !next_staged && bt + 1 < nb) {
            stage_batch(sh, buf ^ 1, bt + 1, total, items, x, n);
        }
        next_staged = true;
        const long long c_w = walk_clock();
        __syncthreads();
        const long long c_w1 = walk_clock();
        c_wait += c_w1 - c_w;
        if (sh.cmd[round & 1][0] == CMD_SPAN) {
            const long long c_s = walk_clock();
            const int64_t e0 = (int64_t)sh.cmd[round & 1][1] * LEAF;
            const int64_t e1 = min(n, e0 + (int64_t)sh.cmd[round & 1][2] * LEAF);
            const float s = coop_chain(x, e0, e1, __int_as_float(bits), sh.chain);
            if (warp == 0) {
                bits = __float_as_int(s);
                i++;
                n_span++;
                n_span_leaves += sh.cmd[round & 1][2];
                c_span += walk_clock() - c_s;
            }
            continue;  // same batch, next item
        }
        bt++;
        next_staged = false;
        c_post += walk_clock() - c_w1;
    }
    if (tid == 0) {
        out[0] = __fmul_rn(factor, __int_as_float(bits));
        hdr->stats[0] = total;
        hdr->stats[1] = counts.applied;  // counted in diagnostic builds only
        hdr->stats[2] = counts.leaves;
        hdr->stats[3] = n_span;
        hdr->stats[4] = n_span_leaves;
        hdr->stats[5] = counts.soft_fail;
        hdr->stats[6] = n_run_fail;
        hdr->stats[7] = walk_clock() - c_begin;
        hdr->stats[8] = c_items;  // includes c_raw
        hdr->stats[9] = c_raw;
        hdr->stats[10] = c_span + (c_pre << 32);
        hdr->stats[11] = c_wait + (c_post << 32);
    }
}

// Short chains: one thread walks shared-memory tiles that the rest of the CTA stages.
__global__ void __launch_bounds__(256)
short_chain_kernel(const float *__restrict__ x, float *__restrict__ out, int64_t n, float factor)
{
    __shared__ __align__(16) float buf[2 * CHAIN_TILE];
    const float s = coop_chain(x, 0, n, 0.0f, buf);
    if (threadIdx.x == 0) out[0] = __fmul_rn(factor, s);
}

constexpr int64_t kShortChain = 1 << 16;  // below this the plain walk is faster than six launches

struct Layout {
    int64_t nnodes;
    long long cap;
    size_t off_hdr, off_tile, off_node, off_pred, off_rabs, off_rec, off_items, total;
};

constexpr size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }

constexpr Layout layout_for(int64_t n)
{
    Layout L{};
    L.nnodes = (n + NODE - 1) / NODE;
    L.cap = 24 * (long long)L.nnodes + 32768;  // = s1::item_capacity(nnodes)
    size_t o = 0;
    L.off_hdr = o;   o = up256(o + sizeof(Header));
    L.off_tile = o;  o = up256(o + (size_t)L.nnodes * TILES_PER_NODE * sizeof(double));
    L.off_node = o;  o = up256(o + (size_t)L.nnodes * sizeof(double));
    L.off_pred = o;  o = up256(o + (size_t)L.nnodes * sizeof(double));
    L.off_rabs = o;  o = up256(o + (size_t)L.nnodes * sizeof(double));
    L.off_rec = o;   o = up256(o + (size_t)L.nnodes * sizeof(NodeRec));
    L.off_items = o; o = up256(o + (size_t)L.cap * sizeof(Item));
    L.total = o;
    return L;
}

}  // namespace

int sum1d_plain(const float *x, float *out, int64_t n, float factor, cudaStream_t st)
{
    short_chain_kernel<<<1, 256, 0, st>>>(x, out, n, factor);
    return launch_status();
}

}  // namespace repdl_b200

using namespace repdl_b200;

extern "C" size_t repdl_b200_sum1d_scratch_bytes(int64_t n)
{
    if (n < kShortChain) return 0;
    return layout_for(n).total;
}

// Opt-in to the walk kernel's dynamic shared memory on the current device (once per device).
static int walk_kernel_ready()
{
    static unsigned long long smem_done = 0;
    return ensure_smem(walk_kernel, WALK_SMEM_BYTES, &smem_done);
}

// The six launches of a long chain on scratch memory `base` (device address, 256-byte aligned, at
// least layout_for(n).total bytes).  Nothing in the scratch has to be initialised: every word that
// is read has been written earlier in the same call.
static int sum1d_long(const float *x, float *out, int64_t n, float factor, char *base, cudaStream_t st)
{
    const Layout L = layout_for(n);
    if (L.nnodes * LEAVES_PER_NODE > 0x7FFFFFFF) return REPDL_E_RANGE;  // leaf indices are 32-bit
    Header *hdr = reinterpret_cast<Header *>(base + L.off_hdr);
    double *tile_sum = reinterpret_cast<double *>(base + L.off_tile);
    double *node_sum = reinterpret_cast<double *>(base + L.off_node);
    double *pred = reinterpret_cast<double *>(base + L.off_pred);
    double *rabs = reinterpret_cast<double *>(base + L.off_rabs);
    NodeRec *rec = reinterpret_cast<NodeRec *>(base + L.off_rec);
    Item *items = reinterpret_cast<Item *>(base + L.off_items);
    const int vec = aligned16(x) ? 1 : 0;
    const unsigned nn = (unsigned)L.nnodes;
    int e;
    if ((e = walk_kernel_ready())) return e;
    tile_sum_kernel<<<nn, 256, 0, st>>>(x, n, tile_sum, node_sum, vec);
    if ((e = launch_status())) return e;
    predict_kernel<<<1, 1024, 0, st>>>(node_sum, (int)nn, pred, rabs);
    if ((e = launch_status())) return e;
    classify_kernel<<<nn, 256, 0, st>>>(x, n, tile_sum, pred, rabs, rec, vec);
    if ((e = launch_status())) return e;
    plan_kernel<<<1, 1024, 0, st>>>(rec, (int)nn, L.cap, hdr, items);
    if ((e = launch_status())) return e;
    const unsigned emit_grid = nn;  // one node per CTA (smooth nodes: one item each, written by thread 0)
    emit_kernel<<<emit_grid, EMIT_WARPS * 32, 0, st>>>(x, n, tile_sum, pred, rabs, rec, items, hdr, vec, L.nnodes);
    if ((e = launch_status())) return e;
    walk_kernel<<<1, WALK_THREADS, WALK_SMEM_BYTES, st>>>(x, n, hdr, items, factor, out);
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

// What the last long-chain call on `scratch` did (after that call has finished on the device):
// copies the walker's counters -- items in the stream, summaries applied, leaves walked with real
// adds, spans walked with real adds and their leaves, composed soft runs that did not fit, composed
// robust runs that did not fit, and (diagnostic builds) the walker's cycle counters -- into
// stats[0..12) on the host.  Diagnostics for benchmarks.
extern "C" int repdl_b200_sum1d_stats(const void *scratch, long long *stats)
{
    if (!scratch || !stats) return REPDL_E_NULL;
    Header h;
    cudaError_t e = cudaMemcpy(&h, scratch, sizeof(Header), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return (int)e;
    for (int k = 0; k < 12; k++) stats[k] = h.stats[k];
    return 0;
}

// ------------------------------------------------------------------------------------------------
// The same chain sum for callers that must not allocate: the scratch is a fixed array in this
// library's device image instead of a buffer the caller provides.
// ------------------------------------------------------------------------------------------------
namespace {
constexpr int64_t kStaticMaxN = (int64_t)1 << 28;                      // 2^28 elements (1 GiB of input)
constexpr size_t kStaticScratchBytes = layout_for(kStaticMaxN).total;  // about 10 MB
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
    // The per-device set-up comes first, whatever the length, so that any first call on a device
    // does it (and a caller who warms up before a stream capture has it behind them).
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
        int e = walk_kernel_ready();
        if (e) return e;
        __atomic_store_n(&g_static_scratch_addr[dev], addr, __ATOMIC_RELEASE);
    }
    if (n < kShortChain) return sum1d_plain(x, out, n, factor, st);
    // nothing in the scratch needs clearing: each call writes every word before reading it
    return sum1d_long(x, out, n, factor, static_cast<char *>(addr), st);
}
