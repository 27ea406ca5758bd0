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
//
// The inner product runs on Blackwell's packed FP32 FMA, fma.rn.f32x2: one instruction performs two
// independent IEEE single-rounding FMAs on a 64-bit register pair -- the same bits as two scalar
// FFMAs, in half the issue slots, which leaves room for the shared-memory loads without starving
// the FMA pipe.  Accumulators live as (j, j+1) column pairs; the B fragment arrives as pairs from
// LDS.128; the A slab is stored in shared memory with every value DUPLICATED, so that the (a, a)
// broadcast pair also arrives straight from LDS.128 with no register moves.
#include "common.cuh"

namespace repdl_b200 {
namespace {

#ifndef REPDL_MM_BK
#define REPDL_MM_BK 16
#endif
#ifndef REPDL_MM_MINB_BIG
#define REPDL_MM_MINB_BIG 1
#endif
#ifndef REPDL_MM_KUNROLL
#define REPDL_MM_KUNROLL REPDL_MM_BK  // k-steps of a slab unrolled back to back
#endif
#ifndef REPDL_MM_GROUP
#define REPDL_MM_GROUP 8
#endif
#define REPDL_PRAGMA(x) _Pragma(#x)
#define REPDL_UNROLL(n) REPDL_PRAGMA(unroll n)
constexpr int BK = REPDL_MM_BK;

// Cooperative loader for one operand slab of BX (rows or columns of C) x BK (k).
//   KCONTIG = true : element (x, k) lives at X[x * ld + k]   (A of a plain mm, B of transB)
//   KCONTIG = false: element (x, k) lives at X[k * ld + x]   (B of a plain mm, A of transA)
//   VEC            : 128-bit global loads (caller guarantees 16 B alignment of every group)
//   DUP            : every value is written twice, S[k][2x] = S[k][2x+1] (the A operand)
// Shared layout is always S[k][x] (S[k][2x], S[k][2x+1] when DUP) with a padded row pitch.
template <int BX, int NT, bool KCONTIG, bool VEC, bool DUP>
struct SlabLoader {
    static constexpr int NV = BX * BK / 4 / NT;
    static constexpr int PITCH = (DUP ? 2 * BX : BX) + 4;
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
                if (DUP) {
                    *reinterpret_cast<float2 *>(&S[k + 0][2 * x]) = make_float2(v[i].x, v[i].x);
                    *reinterpret_cast<float2 *>(&S[k + 1][2 * x]) = make_float2(v[i].y, v[i].y);
                    *reinterpret_cast<float2 *>(&S[k + 2][2 * x]) = make_float2(v[i].z, v[i].z);
                    *reinterpret_cast<float2 *>(&S[k + 3][2 * x]) = make_float2(v[i].w, v[i].w);
                } else {
                    S[k + 0][x] = v[i].x;
                    S[k + 1][x] = v[i].y;
                    S[k + 2][x] = v[i].z;
                    S[k + 3][x] = v[i].w;
                }
            } else {
                int k = idx / (BX / 4);
                int x = (idx % (BX / 4)) * 4;
                if (DUP) {
                    *reinterpret_cast<float4 *>(&S[k][2 * x]) =
                        make_float4(v[i].x, v[i].x, v[i].y, v[i].y);
                    *reinterpret_cast<float4 *>(&S[k][2 * x + 4]) =
                        make_float4(v[i].z, v[i].z, v[i].w, v[i].w);
                } else {
                    *reinterpret_cast<float4 *>(&S[k][x]) = v[i];
                }
            }
        }
    }
};

// Maps the linear CTA index to a C tile so that consecutive CTAs share A and B panels in L2:
// tiles are visited in groups of GROUP tile-rows, column by column inside a group.
__device__ __forceinline__ void tile_of_cta(int pid, int tilesM, int tilesN, int &tm, int &tn)
{
    constexpr int GROUP = REPDL_MM_GROUP;
    int per_group = GROUP * tilesN;
    int g = pid / per_group;
    int first = g * GROUP;
    int gsz = min(tilesM - first, GROUP);
    int r = pid - g * per_group;
    tm = first + r % gsz;
    tn = r / gsz;
}

// Where a finished C tile goes: to one matrix, or -- for the row-sharded multi-GPU product -- to the
// same rows of the C buffers of all ranks of the node (peer pointers over NVLink), so that the
// all-gather happens tile by tile inside the GEMM epilogue instead of as a separate collective.
constexpr int kMaxRanks = 8;
struct OutSet {
    float *p[kMaxRanks];
    int n;
};

// Thread tile TM x TN (multiples of 4): TM/4 row quads and TN/4 column quads, quad q of a thread
// sitting q * (tile extent / quads) apart, so that the 8 lanes of a warp that differ in their
// column read 8 consecutive 16-byte groups of a shared-memory row (no bank conflicts) and lanes that
// share a row or a column get their fragment by broadcast.
#ifndef REPDL_MM_F2
#define REPDL_MM_F2 0   // 1: inner product on the packed fma.rn.f32x2 (same bits; measured slower)
#endif
#ifndef REPDL_MM_ORDER
#define REPDL_MM_ORDER 0
#endif
constexpr bool kF2 = REPDL_MM_F2 != 0;

template <int BM, int BN, int TM, int TN, bool A_KC, bool B_KC, bool VEC, int MINB, int D>
__global__ void __launch_bounds__((BM / TM) * (BN / TN), MINB)
sgemm_kernel(const float *__restrict__ A, const float *__restrict__ B, const OutSet out, int M,
             int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int tilesM, int tilesN, int vecC)
{
    constexpr int NT = (BM / TM) * (BN / TN);
    constexpr int QM = TM / 4, QN = TN / 4;
    constexpr int WX = (BN / TN) / 8;  // warps along n; a warp is 8 lanes along n x 4 along m
    using LoadA = SlabLoader<BM, NT, A_KC, VEC, kF2>;
    using LoadB = SlabLoader<BN, NT, B_KC, VEC, false>;
    constexpr int PA = LoadA::PITCH, PB = LoadB::PITCH;
    extern __shared__ __align__(16) float smem[];
    float(*As)[BK][PA] = reinterpret_cast<float(*)[BK][PA]>(smem);
    float(*Bs)[BK][PB] = reinterpret_cast<float(*)[BK][PB]>(smem + 2 * BK * PA);

    int tm, tn;
    tile_of_cta(blockIdx.x, tilesM, tilesN, tm, tn);
    const int m0 = tm * BM, n0 = tn * BN;
    const int t = threadIdx.x;
    const int lane = t & 31, wid = t >> 5;
    const int tx = (wid % WX) * 8 + (lane & 7);
    const int ty = (wid / WX) * 4 + (lane >> 3);

    float acc[TM][TN];                   // scalar mode
    unsigned long long acc2[TM][TN / 2];  // packed mode: columns (2p, 2p+1) of row i
#pragma unroll
    for (int i = 0; i < TM; i++) {
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = 0.0f;
#pragma unroll
        for (int j = 0; j < TN / 2; j++) acc2[i][j] = 0ull;  // (+0.0f, +0.0f)
    }

    // D register sets hold the slabs kt + 1 .. kt + D on their way from global to shared memory.
    // D = 1 is the plain double buffer; a small tile with a long K cannot cover the L2 / HBM latency
    // with the arithmetic of one slab and few CTAs are resident, so it keeps D = 4 slabs in flight.
    LoadA la[D];
    LoadB lb[D];
    const int nk = (K + BK - 1) / BK;
#pragma unroll
    for (int s = 0; s < D; s++) {
        if (s < nk) {
            la[s].load(A, lda, m0, s * BK, M, K, -0.0f, t);
            lb[s].load(B, ldb, n0, s * BK, N, K, 0.0f, t);
        }
    }
    la[0].store(As[0], t);
    lb[0].store(Bs[0], t);
    __syncthreads();

    for (int kt0 = 0; kt0 < nk; kt0 += D) {
#pragma unroll
      for (int s = 0; s < D; s++) {
        const int kt = kt0 + s;
        if (kt >= nk) break;
        const int cur = kt & 1;
        const bool more = kt + 1 < nk;
        // slab kt already sits in shared memory, so its register set takes slab kt + D
        if (kt + D < nk) {
            la[s].load(A, lda, m0, (kt + D) * BK, M, K, -0.0f, t);
            lb[s].load(B, ldb, n0, (kt + D) * BK, N, K, 0.0f, t);
        }
        REPDL_UNROLL(REPDL_MM_KUNROLL)
        for (int k = 0; k < BK; k++) {
            if constexpr (kF2) {
                unsigned long long a[TM], b[TN / 2];  // a[i] = (a_i, a_i); b[p] = (b_2p, b_2p+1)
#pragma unroll
                for (int q = 0; q < QM; q++) {
                    const float *src = &As[cur][k][2 * (q * (BM / QM) + ty * 4)];
                    ulonglong2 v0 = *reinterpret_cast<const ulonglong2 *>(src);
                    ulonglong2 v1 = *reinterpret_cast<const ulonglong2 *>(src + 4);
                    a[q * 4 + 0] = v0.x, a[q * 4 + 1] = v0.y, a[q * 4 + 2] = v1.x, a[q * 4 + 3] = v1.y;
                }
#pragma unroll
                for (int q = 0; q < QN; q++) {
                    ulonglong2 v =
                        *reinterpret_cast<const ulonglong2 *>(&Bs[cur][k][q * (BN / QN) + tx * 4]);
                    b[q * 2 + 0] = v.x, b[q * 2 + 1] = v.y;
                }
#pragma unroll
                for (int i = 0; i < TM; i++)
#pragma unroll
                    for (int j = 0; j < TN / 2; j++)
                        asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc2[i][j]) : "l"(a[i]), "l"(b[j]));
            } else {
                float a[TM], b[TN];
#pragma unroll
                for (int q = 0; q < QM; q++) {
                    float4 v = *reinterpret_cast<const float4 *>(&As[cur][k][q * (BM / QM) + ty * 4]);
                    a[q * 4 + 0] = v.x, a[q * 4 + 1] = v.y, a[q * 4 + 2] = v.z, a[q * 4 + 3] = v.w;
                }
#pragma unroll
                for (int q = 0; q < QN; q++) {
                    float4 v = *reinterpret_cast<const float4 *>(&Bs[cur][k][q * (BN / QN) + tx * 4]);
                    b[q * 4 + 0] = v.x, b[q * 4 + 1] = v.y, b[q * 4 + 2] = v.z, b[q * 4 + 3] = v.w;
                }
#if REPDL_MM_ORDER == 0
#pragma unroll
                for (int i = 0; i < TM; i++)
#pragma unroll
                    for (int j = 0; j < TN; j++) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
#else
#pragma unroll
                for (int j = 0; j < TN; j++)
#pragma unroll
                    for (int i = 0; i < TM; i++) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
#endif
            }
        }
        if (more) {
            la[(s + 1) % D].store(As[cur ^ 1], t);
            lb[(s + 1) % D].store(Bs[cur ^ 1], t);
        }
        __syncthreads();
      }
    }

#pragma unroll
    for (int i = 0; i < TM; i++) {
        int row = m0 + (i / 4) * (BM / QM) + ty * 4 + (i % 4);
        if (row >= M) continue;
#pragma unroll
        for (int q = 0; q < QN; q++) {
            int col = n0 + q * (BN / QN) + tx * 4;
            float c[4];
            if constexpr (kF2) {
                asm("mov.b64 {%0,%1}, %2;" : "=f"(c[0]), "=f"(c[1]) : "l"(acc2[i][q * 2 + 0]));
                asm("mov.b64 {%0,%1}, %2;" : "=f"(c[2]), "=f"(c[3]) : "l"(acc2[i][q * 2 + 1]));
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++) c[j] = acc[i][q * 4 + j];
            }
            for (int r = 0; r < out.n; r++) {
                float *crow = out.p[r] + (int64_t)row * ldc;
                if (vecC) {
                    if (col < N)
                        *reinterpret_cast<float4 *>(crow + col) = make_float4(c[0], c[1], c[2], c[3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        if (col + j < N) crow[col + j] = c[j];
                }
            }
        }
    }
}

template <int BM, int BN, int TM, int TN, bool A_KC, bool B_KC, bool VEC, int MINB, int D = 1>
int launch_one(const float *A, const float *B, const OutSet &C, int M, int N, int K, int64_t lda,
               int64_t ldb, int64_t ldc, int vecC, cudaStream_t st)
{
    int tilesM = (M + BM - 1) / BM, tilesN = (N + BN - 1) / BN;
    int64_t tiles = (int64_t)tilesM * tilesN;
    if (tiles > 0x7FFFFFFF) return REPDL_E_RANGE;
    auto kern = sgemm_kernel<BM, BN, TM, TN, A_KC, B_KC, VEC, MINB, D>;
    constexpr int smem_bytes = 2 * BK * ((kF2 ? 2 : 1) * BM + 4 + BN + 4) * (int)sizeof(float);
    static unsigned long long smem_done = 0;  // one mask per kernel instantiation
    int e = ensure_smem(kern, smem_bytes, &smem_done);
    if (e) return e;
    kern<<<(unsigned)tiles, (BM / TM) * (BN / TN), smem_bytes, st>>>(A, B, C, M, N, K, lda, ldb, ldc,
                                                                      tilesM, tilesN, vecC);
    return launch_status();
}

#ifndef REPDL_MM_BM
#define REPDL_MM_BM 128
#define REPDL_MM_BN 256
#define REPDL_MM_TM 8
#define REPDL_MM_TN 16
#endif
#define REPDL_MM_BIG REPDL_MM_BM, REPDL_MM_BN, REPDL_MM_TM, REPDL_MM_TN
#ifndef REPDL_MM_ALT
#define REPDL_MM_ALT 1   // 0: never use the 192 x 128 configuration
#endif

template <bool A_KC, bool B_KC, bool VEC>
int launch_shape(const float *A, const float *B, const OutSet &C, int M, int N, int K, int64_t lda,
                 int64_t ldb, int64_t ldc, int vecC, cudaStream_t st)
{
    // Big tiles once they fill the machine twice over; small tiles otherwise so that a
    // 1024 x 1024 problem still spreads over all 148 SMs.  Two big configurations: 192 x 128 with
    // 12 x 8 outputs per thread runs 3 % faster per FMA than 128 x 256 with 8 x 16 (its unrolled slab
    // fits the instruction cache), but which one finishes first also depends on how the tile count
    // rounds up to whole waves and how much of the edge tiles is padding, so both are costed.
    const int64_t sms = sm_count();
    const int64_t tiles_a = (int64_t)((M + 191) / 192) * ((N + 127) / 128);
    const int64_t tiles_b = (int64_t)((M + REPDL_MM_BM - 1) / REPDL_MM_BM) * ((N + REPDL_MM_BN - 1) / REPDL_MM_BN);
    if (tiles_a >= 2 * sms || tiles_b >= 2 * sms) {
        const double cost_a = (double)((tiles_a + sms - 1) / sms) * (192.0 * 128.0) / 1.033;
        const double cost_b = (double)((tiles_b + sms - 1) / sms) * ((double)REPDL_MM_BM * REPDL_MM_BN);
        if (REPDL_MM_ALT && tiles_a >= 2 * sms && (cost_a < cost_b || tiles_b < 2 * sms))
            return launch_one<192, 128, 12, 8, A_KC, B_KC, VEC, 1>(A, B, C, M, N, K, lda, ldb, ldc, vecC, st);
        return launch_one<REPDL_MM_BIG, A_KC, B_KC, VEC, REPDL_MM_MINB_BIG>(A, B, C, M, N, K, lda,
                                                                           ldb, ldc, vecC, st);
    }
    int64_t mid = (int64_t)((M + 127) / 128) * ((N + 63) / 64);
    if (mid >= 2 * (int64_t)sm_count())
        return launch_one<128, 64, 8, 8, A_KC, B_KC, VEC, 4>(A, B, C, M, N, K, lda, ldb, ldc, vecC,
                                                             st);
    // Few outputs but a long K (e.g. a 256 x 128 layer output over K = 9216): the time is K times
    // the instructions one warp issues per k-step, so spread the outputs over more, thinner CTAs.
    int64_t small = (int64_t)((M + 63) / 64) * ((N + 63) / 64);
    if (small * 4 <= (int64_t)sm_count() && K >= 1024)
        return launch_one<32, 32, 4, 4, A_KC, B_KC, VEC, 8, 4>(A, B, C, M, N, K, lda, ldb, ldc, vecC, st);
    return launch_one<64, 64, 8, 8, A_KC, B_KC, VEC, 8>(A, B, C, M, N, K, lda, ldb, ldc, vecC, st);
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

static int mm_dispatch(const float *A, const float *B, const OutSet &out, int64_t M, int64_t N,
                       int64_t K, int transA, int transB, int64_t lda, int64_t ldb, int64_t ldc,
                       void *stream)
{
    if (M < 0 || N < 0 || K < 0) return REPDL_E_SHAPE;
    if (M == 0 || N == 0) return REPDL_OK;
    for (int r = 0; r < out.n; r++)
        if (!out.p[r]) return REPDL_E_NULL;
    if (K > 0 && (!A || !B)) return REPDL_E_NULL;
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
    int vecC = ldc % 4 == 0 && N % 4 == 0;
    for (int r = 0; r < out.n; r++) vecC = vecC && aligned16(out.p[r]);
    const int m = (int)M, n = (int)N, k = (int)K;
#define REPDL_MM_CASE(AKC, BKC)                                                              \
    (vec ? launch_shape<AKC, BKC, true>(A, B, out, m, n, k, lda, ldb, ldc, vecC, st)         \
         : launch_shape<AKC, BKC, false>(A, B, out, m, n, k, lda, ldb, ldc, vecC, st))
    if (a_kc && !b_kc) return REPDL_MM_CASE(true, false);
    if (a_kc && b_kc) return REPDL_MM_CASE(true, true);
    if (!a_kc && !b_kc) return REPDL_MM_CASE(false, false);
    return REPDL_MM_CASE(false, true);
#undef REPDL_MM_CASE
}

extern "C" int repdl_b200_mm(const float *A, const float *B, float *C, int64_t M, int64_t N,
                             int64_t K, int transA, int transB, int64_t lda, int64_t ldb,
                             int64_t ldc, void *stream)
{
    clear_stale_error();
    OutSet out{};
    out.p[0] = C;
    out.n = 1;
    return mm_dispatch(A, B, out, M, N, K, transA, transB, lda, ldb, ldc, stream);
}

extern "C" int repdl_b200_mm_allgather(const float *A_rows, const float *B, float *const *C_of_rank,
                                       int nranks, int64_t row0, int64_t M_local, int64_t N,
                                       int64_t K, int transA, int transB, int64_t lda, int64_t ldb,
                                       int64_t ldc, void *stream)
{
    clear_stale_error();
    if (nranks < 1 || nranks > kMaxRanks || row0 < 0) return REPDL_E_SHAPE;
    if (!C_of_rank) return REPDL_E_NULL;
    OutSet out{};
    out.n = nranks;
    for (int r = 0; r < nranks; r++) {
        if (!C_of_rank[r]) return REPDL_E_NULL;
        out.p[r] = C_of_rank[r] + row0 * ldc;
    }
    return mm_dispatch(A_rows, B, out, M_local, N, K, transA, transB, lda, ldb, ldc, stream);
}
