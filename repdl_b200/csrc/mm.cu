// Bit-reproducible fp32 matrix multiplication for sm_100a.
//
// Contract (microsoft/RepDL backend/cpu/matrix_multiplication.cpp:26-33): every output element is
// ONE fp32 accumulator that starts at +0 and receives fmaf(a_k, b_k, acc) for k = 0, 1, ..., K-1 in
// that order.  The kernel below is a register-blocked SIMT SGEMM on the FP32 FMA pipe: tensor
// cores are deliberately not used because the accumulation order and intermediate rounding of
// tcgen05.mma are not specified bit for bit.  Parallelism comes only from the M x N output
// elements; K is walked sequentially by the single thread that owns the element, so the result
// does not depend on tile shape, grid size or GPU count.
//
// Structure: C tile BM x BN per CTA, 8 x 8 outputs per thread (as two 4-wide halves in each
// direction so that fragments are read with conflict-free LDS.128), K walked in slabs of 16 that
// are staged global -> registers -> shared memory (double buffered; the register stage lets a
// k-contiguous operand be transposed on the way in, so all four transpose variants share one
// inner loop).  The slab that holds the K tail is padded with A = -0.0f, B = +0.0f: the padded
// product is -0, and acc + (-0) == acc for EVERY acc including -0, +0, inf and NaN, so the padded
// steps are exact identities (a +0 pad would turn an accumulator of -0 into +0).
#include "common.cuh"

namespace repdl_b200 {
namespace {

constexpr int BK = 16;

// Cooperative loader for one operand slab of BX (rows or columns of C) x BK (k).
//   KCONTIG = true : element (x, k) lives at X[x * ld + k]   (A of a plain mm, B of transB)
//   KCONTIG = false: element (x, k) lives at X[k * ld + x]   (B of a plain mm, A of transA)
//   VEC            : 128-bit global loads (caller guarantees 16 B alignment of every group)
// Shared layout is always S[k][x] with row pitch BX + 4.
template <int BX, int NT, bool KCONTIG, bool VEC>
struct SlabLoader {
    static constexpr int NV = BX * BK / 4 / NT;
    static constexpr int PITCH = BX + 4;
    float4 v[NV];

    __device__ __forceinline__ void load(const float *__restrict__ X, int64_t ld, int x0, int k0,
                                         int xmax, int kmax, float pad, int t)
    {
#pragma unroll
        for (int i = 0; i < NV; i++) {
            int idx = t + NT * i;
            if (KCONTIG) {
                int x = x0 + idx / (BK / 4);
                int k = k0 + (idx % (BK / 4)) * 4;
                const float *p = X + (int64_t)x * ld + k;
                if (VEC) {
                    v[i] = (x < xmax && k < kmax) ? ldg_f4(p) : make_float4(pad, pad, pad, pad);
                } else {
                    bool xin = x < xmax;
                    v[i].x = (xin && k + 0 < kmax) ? __ldg(p + 0) : pad;
                    v[i].y = (xin && k + 1 < kmax) ? __ldg(p + 1) : pad;
                    v[i].z = (xin && k + 2 < kmax) ? __ldg(p + 2) : pad;
                    v[i].w = (xin && k + 3 < kmax) ? __ldg(p + 3) : pad;
                }
            } else {
                int k = k0 + idx / (BX / 4);
                int x = x0 + (idx % (BX / 4)) * 4;
                const float *p = X + (int64_t)k * ld + x;
                if (VEC) {
                    v[i] = (x < xmax && k < kmax) ? ldg_f4(p) : make_float4(pad, pad, pad, pad);
                } else {
                    bool kin = k < kmax;
                    v[i].x = (kin && x + 0 < xmax) ? __ldg(p + 0) : pad;
                    v[i].y = (kin && x + 1 < xmax) ? __ldg(p + 1) : pad;
                    v[i].z = (kin && x + 2 < xmax) ? __ldg(p + 2) : pad;
                    v[i].w = (kin && x + 3 < xmax) ? __ldg(p + 3) : pad;
                }
            }
        }
    }

    __device__ __forceinline__ void store(float (*S)[PITCH], int t) const
    {
#pragma unroll
        for (int i = 0; i < NV; i++) {
            int idx = t + NT * i;
            if (KCONTIG) {
                int x = idx / (BK / 4);
                int k = (idx % (BK / 4)) * 4;
                S[k + 0][x] = v[i].x;
                S[k + 1][x] = v[i].y;
                S[k + 2][x] = v[i].z;
                S[k + 3][x] = v[i].w;
            } else {
                int k = idx / (BX / 4);
                int x = (idx % (BX / 4)) * 4;
                *reinterpret_cast<float4 *>(&S[k][x]) = v[i];
            }
        }
    }
};

// Maps the linear CTA index to a C tile so that consecutive CTAs share A and B panels in L2:
// tiles are visited in groups of GROUP tile-rows, column by column inside a group.
__device__ __forceinline__ void tile_of_cta(int pid, int tilesM, int tilesN, int &tm, int &tn)
{
    constexpr int GROUP = 8;
    int per_group = GROUP * tilesN;
    int g = pid / per_group;
    int first = g * GROUP;
    int gsz = min(tilesM - first, GROUP);
    int r = pid - g * per_group;
    tm = first + r % gsz;
    tn = r / gsz;
}

template <int BM, int BN, bool A_KC, bool B_KC, bool VEC, int MINB>
__global__ void __launch_bounds__((BM / 8) * (BN / 8), MINB)
sgemm_kernel(const float *__restrict__ A, const float *__restrict__ B, float *__restrict__ C,
             int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int tilesM, int tilesN,
             int vecC)
{
    constexpr int NT = (BM / 8) * (BN / 8);
    constexpr int WX = BN / 64;  // warps along n (a warp spans 8 threads = 32 + 32 columns)
    using LoadA = SlabLoader<BM, NT, A_KC, VEC>;
    using LoadB = SlabLoader<BN, NT, B_KC, VEC>;
    __shared__ __align__(16) float As[2][BK][LoadA::PITCH];
    __shared__ __align__(16) float Bs[2][BK][LoadB::PITCH];

    int tm, tn;
    tile_of_cta(blockIdx.x, tilesM, tilesN, tm, tn);
    const int m0 = tm * BM, n0 = tn * BN;
    const int t = threadIdx.x;
    const int lane = t & 31, wid = t >> 5;
    const int tx = (wid % WX) * 8 + (lane & 7);
    const int ty = (wid / WX) * 4 + (lane >> 3);
    const int c0 = tx * 4, c1 = BN / 2 + tx * 4;
    const int r0 = ty * 4, r1 = BM / 2 + ty * 4;

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;

    LoadA la;
    LoadB lb;
    const int nk = (K + BK - 1) / BK;
    la.load(A, lda, m0, 0, M, K, -0.0f, t);
    lb.load(B, ldb, n0, 0, N, K, 0.0f, t);
    la.store(As[0], t);
    lb.store(Bs[0], t);
    __syncthreads();

    for (int kt = 0; kt < nk; kt++) {
        const int cur = kt & 1;
        const bool more = kt + 1 < nk;
        if (more) {
            la.load(A, lda, m0, (kt + 1) * BK, M, K, -0.0f, t);
            lb.load(B, ldb, n0, (kt + 1) * BK, N, K, 0.0f, t);
        }
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float4 a0 = *reinterpret_cast<const float4 *>(&As[cur][k][r0]);
            float4 a1 = *reinterpret_cast<const float4 *>(&As[cur][k][r1]);
            float4 b0 = *reinterpret_cast<const float4 *>(&Bs[cur][k][c0]);
            float4 b1 = *reinterpret_cast<const float4 *>(&Bs[cur][k][c1]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
        }
        if (more) {
            la.store(As[cur ^ 1], t);
            lb.store(Bs[cur ^ 1], t);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 8; i++) {
        int row = m0 + (i < 4 ? r0 + i : r1 + i - 4);
        if (row >= M) continue;
        float *crow = C + (int64_t)row * ldc;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            int col = n0 + (h ? c1 : c0);
            if (vecC) {
                if (col < N)
                    *reinterpret_cast<float4 *>(crow + col) =
                        make_float4(acc[i][h * 4 + 0], acc[i][h * 4 + 1], acc[i][h * 4 + 2],
                                    acc[i][h * 4 + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (col + j < N) crow[col + j] = acc[i][h * 4 + j];
            }
        }
    }
}

template <int BM, int BN, bool A_KC, bool B_KC, bool VEC, int MINB>
int launch_one(const float *A, const float *B, float *C, int M, int N, int K, int64_t lda,
               int64_t ldb, int64_t ldc, int vecC, cudaStream_t st)
{
    int tilesM = (M + BM - 1) / BM, tilesN = (N + BN - 1) / BN;
    int64_t tiles = (int64_t)tilesM * tilesN;
    if (tiles > 0x7FFFFFFF) return REPDL_E_RANGE;
    sgemm_kernel<BM, BN, A_KC, B_KC, VEC, MINB>
        <<<(unsigned)tiles, (BM / 8) * (BN / 8), 0, st>>>(A, B, C, M, N, K, lda, ldb, ldc, tilesM,
                                                           tilesN, vecC);
    return launch_status();
}

template <bool A_KC, bool B_KC, bool VEC>
int launch_shape(const float *A, const float *B, float *C, int M, int N, int K, int64_t lda,
                 int64_t ldb, int64_t ldc, int vecC, cudaStream_t st)
{
    // Big tiles once they fill the machine twice over; small tiles otherwise so that a
    // 1024 x 1024 problem still spreads over all 148 SMs.
    int64_t big = (int64_t)((M + 127) / 128) * ((N + 127) / 128);
    if (big >= 2 * (int64_t)sm_count())
        return launch_one<128, 128, A_KC, B_KC, VEC, 2>(A, B, C, M, N, K, lda, ldb, ldc, vecC, st);
    int64_t mid = (int64_t)((M + 127) / 128) * ((N + 63) / 64);
    if (mid >= 2 * (int64_t)sm_count())
        return launch_one<128, 64, A_KC, B_KC, VEC, 4>(A, B, C, M, N, K, lda, ldb, ldc, vecC, st);
    return launch_one<64, 64, A_KC, B_KC, VEC, 8>(A, B, C, M, N, K, lda, ldb, ldc, vecC, st);
}

}  // namespace

int sm_count()
{
    static thread_local int cached_dev = -1, cached = kNumSMsB200;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return kNumSMsB200;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            cached = n;
        cached_dev = dev;
    }
    return cached;
}

}  // namespace repdl_b200

using namespace repdl_b200;

extern "C" int repdl_b200_mm(const float *A, const float *B, float *C, int64_t M, int64_t N,
                             int64_t K, int transA, int transB, int64_t lda, int64_t ldb,
                             int64_t ldc, void *stream)
{
    if (M < 0 || N < 0 || K < 0) return REPDL_E_SHAPE;
    if (M == 0 || N == 0) return REPDL_OK;
    if (!C || (K > 0 && (!A || !B))) return REPDL_E_NULL;
    if (M > 0x7FFFFFF0 || N > 0x7FFFFFF0 || K > 0x7FFFFFF0) return REPDL_E_RANGE;
    const bool a_kc = !transA, b_kc = transB != 0;
    // smallest legal pitches
    if (lda < (a_kc ? K : M) || ldb < (b_kc ? K : N) || ldc < N) return REPDL_E_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    // 128-bit loads need every 4-element group to be fully inside or fully outside the matrix
    // and 16-byte aligned.
    const bool vecA = aligned16(A) && lda % 4 == 0 && (a_kc ? K : M) % 4 == 0;
    const bool vecB = aligned16(B) && ldb % 4 == 0 && (b_kc ? K : N) % 4 == 0;
    const bool vec = vecA && vecB;
    const int vecC = aligned16(C) && ldc % 4 == 0 && N % 4 == 0;
    const int m = (int)M, n = (int)N, k = (int)K;
#define REPDL_MM_CASE(AKC, BKC)                                                              \
    (vec ? launch_shape<AKC, BKC, true>(A, B, C, m, n, k, lda, ldb, ldc, vecC, st)           \
         : launch_shape<AKC, BKC, false>(A, B, C, m, n, k, lda, ldb, ldc, vecC, st))
    if (a_kc && !b_kc) return REPDL_MM_CASE(true, false);
    if (a_kc && b_kc) return REPDL_MM_CASE(true, true);
    if (!a_kc && !b_kc) return REPDL_MM_CASE(false, false);
    return REPDL_MM_CASE(false, true);
#undef REPDL_MM_CASE
}
