// Fixed-order fp32 sums for sm_100a.
//
// Contract (microsoft/RepDL backend/cpu/summation.cpp:12-78): each result is ONE fp32 accumulator
// that starts at +0 and receives the elements strictly left to right with a rounded fp32 add after
// every element; the mean variants multiply the finished sum once by float(1.0/count).  There is no
// tree: the chain itself is the specification, so a sum is parallel only across independent chains
// (rows, columns, channels).  No atomics anywhere.
#include "common.cuh"

namespace repdl_b200 {
namespace {

// ------------------------------------------------------------------------------------------------
// sum2d_dim1: one chain per row.  One thread owns one row and walks it with 128-bit loads; the 32
// rows of a warp are 32 separate 128-byte lines per step, each of which stays in L1 until its owner
// has consumed all of it, so every DRAM sector is fetched once.  UNROLL independent loads are kept
// in flight per thread (UNROLL * 16 B * resident threads covers the HBM latency-bandwidth product).
// ------------------------------------------------------------------------------------------------
template <int UNROLL>
__global__ void __launch_bounds__(128)
sum_rows_vec_kernel(const float *__restrict__ x, float *__restrict__ out, int64_t M, int64_t N,
                    float factor)
{
    int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= M) return;
    const float4 *p = reinterpret_cast<const float4 *>(x + row * N);
    const int64_t nv = N >> 2;
    float s = 0.0f;
    int64_t j = 0;
    for (; j + UNROLL <= nv; j += UNROLL) {
        float4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) v[u] = __ldg(p + j + u);
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            s = __fadd_rn(s, v[u].x);
            s = __fadd_rn(s, v[u].y);
            s = __fadd_rn(s, v[u].z);
            s = __fadd_rn(s, v[u].w);
        }
    }
    for (; j < nv; j++) {
        float4 v = __ldg(p + j);
        s = __fadd_rn(s, v.x);
        s = __fadd_rn(s, v.y);
        s = __fadd_rn(s, v.z);
        s = __fadd_rn(s, v.w);
    }
    out[row] = __fmul_rn(factor, s);
}

// Staged variant (the fast path): a warp owns 32 rows.  Per stage it copies a [32 rows x 64 columns]
// block to shared memory with cp.async -- 16 lanes cover 256 contiguous bytes of one row, so DRAM
// sees whole 128-byte lines -- three stages deep, and each lane then walks its own row of the
// block with LDS.128 (row pitch 68 floats: the 8 lanes of a quarter-warp hit 8 different 16-byte
// bank groups).  Warps never synchronise with each other.
constexpr int SR_COLS = 64, SR_PITCH = 68, SR_STAGES = 3, SR_WARPS = 2;
constexpr int SR_SMEM_BYTES = SR_WARPS * SR_STAGES * 32 * SR_PITCH * (int)sizeof(float);

__global__ void __launch_bounds__(SR_WARPS * 32)
sum_rows_staged_kernel(const float *__restrict__ x, float *__restrict__ out, int64_t M, int64_t N,
                       float factor)
{
    extern __shared__ __align__(16) float sr_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row0 = ((int64_t)blockIdx.x * SR_WARPS + warp) * 32;
    if (row0 >= M) return;
    float(*buf)[32][SR_PITCH] =
        reinterpret_cast<float(*)[32][SR_PITCH]>(sr_smem + warp * SR_STAGES * 32 * SR_PITCH);
    const int64_t nst = (N + SR_COLS - 1) / SR_COLS;
    const int sub = lane >> 4, c = (lane & 15) * 4;

    auto issue = [&](int64_t st) {
        if (st < nst) {
            const int64_t col = st * SR_COLS + c;
            if (col < N) {
                float(*dst)[SR_PITCH] = buf[st % SR_STAGES];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    int r = i * 2 + sub;
                    int64_t grow = row0 + r;
                    if (grow >= M) grow = M - 1;  // duplicate the last row; its sum is discarded
                    cp_async_16(&dst[r][c], x + grow * N + col);
                }
            }
        }
        cp_async_commit();
    };

#pragma unroll
    for (int s = 0; s < SR_STAGES - 1; s++) issue(s);
    float acc = 0.0f;
    for (int64_t st = 0; st < nst; st++) {
        issue(st + SR_STAGES - 1);
        cp_async_wait<SR_STAGES - 1>();
        __syncwarp();
        const int64_t left = N - st * SR_COLS;
        const int cnt = left < SR_COLS ? (int)left : SR_COLS;  // multiple of 4
        const float4 *rowp = reinterpret_cast<const float4 *>(buf[st % SR_STAGES][lane]);
        if (cnt == SR_COLS) {
#pragma unroll
            for (int q = 0; q < SR_COLS / 4; q++) {
                float4 v = rowp[q];
                acc = __fadd_rn(acc, v.x);
                acc = __fadd_rn(acc, v.y);
                acc = __fadd_rn(acc, v.z);
                acc = __fadd_rn(acc, v.w);
            }
        } else {
            for (int q = 0; q < cnt / 4; q++) {
                float4 v = rowp[q];
                acc = __fadd_rn(acc, v.x);
                acc = __fadd_rn(acc, v.y);
                acc = __fadd_rn(acc, v.z);
                acc = __fadd_rn(acc, v.w);
            }
        }
        __syncwarp();
    }
    if (row0 + lane < M) out[row0 + lane] = __fmul_rn(factor, acc);
}

__global__ void __launch_bounds__(128)
sum_rows_scalar_kernel(const float *__restrict__ x, float *__restrict__ out, int64_t M, int64_t N,
                       float factor)
{
    int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= M) return;
    const float *p = x + row * N;
    float s = 0.0f;
    for (int64_t j = 0; j < N; j++) s = __fadd_rn(s, __ldg(p + j));
    out[row] = __fmul_rn(factor, s);
}

// ------------------------------------------------------------------------------------------------
// sum2d_dim0: one chain per column; a warp reads 32 adjacent columns of one row per step, which is
// already coalesced.  8 rows are loaded ahead of the adds.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
sum_cols_kernel(const float *__restrict__ x, float *__restrict__ out, int64_t M, int64_t N,
                float factor)
{
    int64_t col = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= N) return;
    const float *p = x + col;
    float s = 0.0f;
    int64_t i = 0;
    for (; i + 8 <= M; i += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) v[u] = __ldg(p + (i + u) * N);
#pragma unroll
        for (int u = 0; u < 8; u++) s = __fadd_rn(s, v[u]);
    }
    for (; i < M; i++) s = __fadd_rn(s, __ldg(p + i * N));
    out[col] = __fmul_rn(factor, s);
}

// ------------------------------------------------------------------------------------------------
// One long chain per CTA (sum4d_dim023: one CTA per channel; sum1d lives in sum1d.cu).  The chain is
// the concatenation of `nseg` contiguous segments of `seglen` floats, segment s starting at
// base + s * segstride.  All threads stage the next TILE chain elements into shared memory while
// thread 0 walks the current tile with LDS.128 + four dependent adds; the walk (4 cycles per
// element, the latency of a dependent FADD) is the critical path.
// ------------------------------------------------------------------------------------------------
constexpr int CHAIN_TILE = 4096;
constexpr int CHAIN_THREADS = 256;

__global__ void __launch_bounds__(CHAIN_THREADS)
chain_sum_kernel(const float *__restrict__ x, float *__restrict__ out, int64_t nseg, int64_t seglen,
                 int64_t segstride, int64_t chain_stride, float factor)
{
    __shared__ __align__(16) float buf[2][CHAIN_TILE];
    const float *base = x + (int64_t)blockIdx.x * chain_stride;
    const int64_t total = nseg * seglen;
    const int64_t ntiles = (total + CHAIN_TILE - 1) / CHAIN_TILE;
    const int t = threadIdx.x;

    // Warp 0 only walks; warps 1..7 stage.  Each staging thread keeps (segment, offset) of its next
    // element and advances them by the stride, so no division is needed per element.
    constexpr int STAGERS = CHAIN_THREADS - 32;
    const int st = t - 32;  // index among the staging threads (negative in warp 0)
    int64_t seg = 0, off = 0;
    if (st >= 0) {
        seg = (nseg == 1) ? 0 : st / seglen;
        off = st - seg * seglen;
    }
    // bring (seg, off) back to 0 <= off < seglen after off moved by less than a few strides
    auto renorm = [&]() {
        if (nseg == 1) return;
        if (seglen >= STAGERS) {
            while (off >= seglen) off -= seglen, seg++;
            while (off < 0) off += seglen, seg--;
        } else {
            int64_t q = off / seglen;
            if (off - q * seglen < 0) q--;
            seg += q;
            off -= q * seglen;
        }
    };
    auto stage = [&](int64_t tile, float *dst) {
        if (st < 0) return;
        const int64_t e0 = tile * CHAIN_TILE;
        for (int i = st; i < CHAIN_TILE; i += STAGERS) {
            dst[i] = (e0 + i < total) ? __ldg(base + seg * segstride + off) : 0.0f;
            off += STAGERS;
            renorm();
        }
        // This thread has moved ceil((CHAIN_TILE - st) / STAGERS) strides; its first element of the next
        // tile is CHAIN_TILE after its first element of this one.
        const int moved = ((CHAIN_TILE - st + STAGERS - 1) / STAGERS) * STAGERS;
        off += CHAIN_TILE - moved;
        renorm();
    };
    float s = 0.0f;
    if (ntiles > 0) stage(0, buf[0]);
    __syncthreads();
    for (int64_t tile = 0; tile < ntiles; tile++) {
        const int cur = (int)(tile & 1);
        if (tile + 1 < ntiles) stage(tile + 1, buf[cur ^ 1]);
        if (t == 0) {
            int64_t left = total - tile * CHAIN_TILE;
            int cnt = left < CHAIN_TILE ? (int)left : CHAIN_TILE;
            const float4 *b4 = reinterpret_cast<const float4 *>(buf[cur]);
            int i = 0;
            // 8 loads ahead of the adds: the walk then runs at the latency of the FADD chain
            for (; i + 32 <= cnt; i += 32) {
                float4 v[8];
#pragma unroll
                for (int u = 0; u < 8; u++) v[u] = b4[(i >> 2) + u];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    s = __fadd_rn(s, v[u].x);
                    s = __fadd_rn(s, v[u].y);
                    s = __fadd_rn(s, v[u].z);
                    s = __fadd_rn(s, v[u].w);
                }
            }
            for (; i + 4 <= cnt; i += 4) {
                float4 v = b4[i >> 2];
                s = __fadd_rn(s, v.x);
                s = __fadd_rn(s, v.y);
                s = __fadd_rn(s, v.z);
                s = __fadd_rn(s, v.w);
            }
            for (; i < cnt; i++) s = __fadd_rn(s, buf[cur][i]);
        }
        __syncthreads();
    }
    if (t == 0) out[blockIdx.x] = __fmul_rn(factor, s);
}

}  // namespace
}  // namespace repdl_b200

using namespace repdl_b200;

extern "C" int repdl_b200_sum2d_dim0(const float *x, float *out, int64_t M, int64_t N, float factor,
                                     void *stream)
{
    clear_stale_error();
    if (M < 0 || N < 0) return REPDL_E_SHAPE;
    if (N == 0) return REPDL_OK;
    if (!out || (M > 0 && !x)) return REPDL_E_NULL;
    int64_t blocks = (N + 127) / 128;
    if (blocks > 0x7FFFFFFF) return REPDL_E_RANGE;
    sum_cols_kernel<<<(unsigned)blocks, 128, 0, (cudaStream_t)stream>>>(x, out, M, N, factor);
    return launch_status();
}

extern "C" int repdl_b200_sum2d_dim1(const float *x, float *out, int64_t M, int64_t N, float factor,
                                     void *stream)
{
    clear_stale_error();
    if (M < 0 || N < 0) return REPDL_E_SHAPE;
    if (M == 0) return REPDL_OK;
    if (!out || (N > 0 && !x)) return REPDL_E_NULL;
    int64_t blocks = (M + 127) / 128;
    if (blocks > 0x7FFFFFFF) return REPDL_E_RANGE;
    if (N % 4 == 0 && aligned16(x) && N >= 2 * SR_COLS) {
        static unsigned long long smem_done = 0;
        int e = ensure_smem(sum_rows_staged_kernel, SR_SMEM_BYTES, &smem_done);
        if (e) return e;
        int64_t b2 = (M + SR_WARPS * 32 - 1) / (SR_WARPS * 32);
        sum_rows_staged_kernel<<<(unsigned)b2, SR_WARPS * 32, SR_SMEM_BYTES, (cudaStream_t)stream>>>(
            x, out, M, N, factor);
    } else if (N % 4 == 0 && aligned16(x))
        sum_rows_vec_kernel<8><<<(unsigned)blocks, 128, 0, (cudaStream_t)stream>>>(x, out, M, N,
                                                                                   factor);
    else
        sum_rows_scalar_kernel<<<(unsigned)blocks, 128, 0, (cudaStream_t)stream>>>(x, out, M, N,
                                                                                    factor);
    return launch_status();
}

extern "C" int repdl_b200_sum4d_dim023(const float *x, float *out, int64_t N, int64_t C, int64_t HW,
                                       float factor, void *stream)
{
    clear_stale_error();
    if (N < 0 || C < 0 || HW < 0) return REPDL_E_SHAPE;
    if (C == 0) return REPDL_OK;
    if (!out || (N * HW > 0 && !x)) return REPDL_E_NULL;
    if (C > 0x7FFFFFFF) return REPDL_E_RANGE;
    chain_sum_kernel<<<(unsigned)C, CHAIN_THREADS, 0, (cudaStream_t)stream>>>(x, out, N, HW, C * HW,
                                                                              HW, factor);
    return launch_status();
}
