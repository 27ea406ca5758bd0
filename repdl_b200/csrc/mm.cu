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
// (Blackwell's packed fma.rn.f32x2 gives the same bits in half the issue slots, but measured slower
// here -- 36-44 against 53 TFLOP/s -- because its operand pairs cost register moves or a duplicated
// shared-memory operand; the scalar FFMA loop below is what ships.)
#include "common.cuh"

namespace repdl_b200 {
namespace {

constexpr int BK = 16;  // k-steps per slab, unrolled back to back


// Cooperative loader for one operand slab of BX (rows or columns of C) x BK (k).
//   KCONTIG = true : element (x, k) lives at X[x * ld + k]   (A of a plain mm, B of transB)
//   KCONTIG = false: element (x, k) lives at X[k * ld + x]   (B of a plain mm, A of transA)
//   VEC            : 128-bit global loads (caller guarantees 16 B alignment of every group)
// Shared layout is always S[k][x] with a padded row pitch.
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
template <int BM, int BN, int TM, int TN, bool A_KC, bool B_KC, bool VEC, int MINB, int D>
__global__ void __launch_bounds__((BM / TM) * (BN / TN), MINB)
sgemm_kernel(const float *__restrict__ A, const float *__restrict__ B, const OutSet out, int M,
             int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int tilesM, int tilesN, int vecC)
{
    constexpr int NT = (BM / TM) * (BN / TN);
    constexpr int QM = TM / 4, QN = TN / 4;
    constexpr int WX = (BN / TN) / 8;  // warps along n; a warp is 8 lanes along n x 4 along m
    using LoadA = SlabLoader<BM, NT, A_KC, VEC>;
    using LoadB = SlabLoader<BN, NT, B_KC, VEC>;
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

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++) {
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = 0.0f;
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
#pragma unroll
        for (int k = 0; k < BK; k++) {
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
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
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
#pragma unroll
            for (int j = 0; j < 4; j++) c[j] = acc[i][q * 4 + j];
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
    constexpr int smem_bytes = 2 * BK * (BM + 4 + BN + 4) * (int)sizeof(float);
    static unsigned long long smem_done = 0;  // one mask per kernel instantiation
    int e = ensure_smem(kern, smem_bytes, &smem_done);
    if (e) return e;
    kern<<<(unsigned)tiles, (BM / TM) * (BN / TN), smem_bytes, st>>>(A, B, C, M, N, K, lda, ldb, ldc,
                                                                      tilesM, tilesN, vecC);
    return launch_status();
}

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
    const int64_t tiles_b = (int64_t)((M + 127) / 128) * ((N + 255) / 256);
    if (tiles_a >= 2 * sms || tiles_b >= 2 * sms) {
        const double cost_a = (double)((tiles_a + sms - 1) / sms) * (192.0 * 128.0) / 1.033;
        const double cost_b = (double)((tiles_b + sms - 1) / sms) * (128.0 * 256.0);
        if (tiles_a >= 2 * sms && (cost_a < cost_b || tiles_b < 2 * sms))
            return launch_one<192, 128, 12, 8, A_KC, B_KC, VEC, 1>(A, B, C, M, N, K, lda, ldb, ldc, vecC, st);
        return launch_one<128, 256, 8, 16, A_KC, B_KC, VEC, 1>(A, B, C, M, N, K, lda, ldb, ldc, vecC, st);
    }
    int64_t mid = (int64_t)((M + 127) / 128) * ((N + 63) / 64);
    if (mid >= 2 * sms)
        return launch_one<128, 64, 8, 8, A_KC, B_KC, VEC, 4>(A, B, C, M, N, K, lda, ldb, ldc, vecC, st);
    // Problems that cannot fill the machine twice: the largest tile that still gives most SMs a CTA.
    // Measured on B200 (1024^3, L2 flushed): 64 x 128 tiles 30.4 TFLOP/s (24.4 when the register
    // budget is cut to four CTAs per SM), 32 x 64 with two slabs in flight 27.2, 128 x 64 25.0,
    // 64 x 64 24.4; 512 x 512 x 4096: 32 x 64 11.9 against 64 x 64 6.8.
    const int64_t wide = (int64_t)((M + 63) / 64) * ((N + 127) / 128);
    if (4 * wide >= 3 * sms)
        return launch_one<64, 128, 8, 8, A_KC, B_KC, VEC, 2>(A, B, C, M, N, K, lda, ldb, ldc, vecC, st);
    // Few outputs but a long K in a layout that the chain kernel (mm_long_k) does not take: the time
    // is K times the instructions one warp issues per k-step, so spread the outputs over more, thinner
    // CTAs.
    const int64_t small = (int64_t)((M + 63) / 64) * ((N + 63) / 64);
    if (small * 4 <= sms && K >= 1024)
        return launch_one<32, 32, 4, 4, A_KC, B_KC, VEC, 8, 4>(A, B, C, M, N, K, lda, ldb, ldc, vecC, st);
    if (4 * small >= 3 * sms)
        return launch_one<64, 64, 8, 8, A_KC, B_KC, VEC, 8>(A, B, C, M, N, K, lda, ldb, ldc, vecC, st);
    return launch_one<32, 64, 4, 8, A_KC, B_KC, VEC, 8, 2>(A, B, C, M, N, K, lda, ldb, ldc, vecC, st);
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
    // Few outputs over a long K with both operands k-contiguous and dense (a layer's forward product
    // x W^T): one chain per thread on the chain kernel of the convolution weight gradient, which this
    // product is (C[m][n] = sum_k A[m][k] B[n][k] is the gradient of a 1 x 1 kernel over one image of
    // 1 x K pixels).  256 x 128 outputs over K = 9216: 0.2 ms on 32 x 32 tiles here, because 64 warps
    // issue all the FMAs.
    if (a_kc && b_kc && out.n == 1 && lda == K && ldb == K && ldc == N && K >= 2048 && K % 4 == 0 &&
        aligned16(A) && (int64_t)((M + 63) / 64) * ((N + 63) / 64) * 4 <= sm_count()) {
        const int e = mm_long_k(A, B, out.p[0], m, n, k, st);
        if (e != REPDL_E_UNSUPPORTED) return e;
    }
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
