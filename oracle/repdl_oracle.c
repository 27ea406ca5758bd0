/*
 * TEST INFRASTRUCTURE -- NOT PART OF THE SHIPPED LIBRARY.
 *
 * CPU restatement, in plain C, of the arithmetic of microsoft/RepDL's CPU
 * operator backend (the reference's own statement of "the right bits").  Only
 * the test-suite, the smoke check and the cpu_baseline / reference leg of
 * bench.py may load this file's shared object; the CUDA library never does.
 *
 * Every function cites the reference lines it restates.  The contract it
 * restates is an evaluation ORDER: one fp32 accumulator per output element,
 * started at +0, updated left to right with a single-rounding fmaf (products)
 * or a plain fp32 add (sums).  Loop nests here are re-blocked for speed, but
 * re-blocking only changes which output element is advanced next, never the
 * order of the updates applied to one accumulator, so the bits are the same.
 *
 * Third-party arithmetic behind the reference that this file restates:
 *   - exp/log: the system libm's double-precision exp()/log() (glibc 2.39 in
 *     the image this was pinned on), called at backend/cpu/math.cpp:16,34, then
 *     rounded to fp32 by the implicit double->float conversion.
 *   - div / sqrt / max / sub / gather: ATen CPU kernels of torch 2.11, called at
 *     repdl/ops.py:98-103,122-123, backend/cpu/softmax.cpp:17,19 and
 *     backend/cpu/cross_entropy.cpp:17,21.  They are single IEEE-754 operations;
 *     the only implementation-defined parts are NaN payloads, restated below as
 *     observed from that torch build (see tests/test_oracle_pin.py).
 *
 * Parity pin: tests/test_oracle_pin.py checks every function here bit for bit
 * against the reference's own CPU backend compiled from its unmodified sources
 * (oracle/_ref, built by oracle/build_ref.sh) when that build is present, and
 * against the fixtures under tests/golden/ (generated from the same build by
 * tests/golden/make_golden.py) everywhere else.
 *
 * Build: gcc -O3 -march=native -ffp-contract=off -fno-fast-math -fopenmp -fPIC -shared
 *        (oracle/build.py).  -ffp-contract=off matters: the only fused
 *        operations allowed are the explicit fmaf() calls.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

typedef int64_t i64;

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------- *
 * mm -- backend/cpu/matrix_multiplication.cpp:12-36
 *   C[i][j] = fold_{k ascending} fmaf(A(i,k), B(k,j), .) from +0,
 *   A(i,k) = transA ? A[k][i] : A[i][k]; B(k,j) = transB ? B[j][k] : B[k][j].
 * Element strides are explicit because the reference reads through accessors
 * (matrix_multiplication.cpp:19-21) and so honours non-contiguous inputs.
 * The loops are tiled (rows x 64 columns x 256 k) with the k tiles visited in
 * ascending order and the accumulators carried in C between k tiles, which is
 * the same chain per element.
 * ------------------------------------------------------------------------- */
#define MM_JT 64
#define MM_KT 256
#define MM_IT 4

void oracle_mm(const float *A, i64 sa0, i64 sa1, const float *B, i64 sb0, i64 sb1,
               float *C, i64 M, i64 N, i64 K, int transA, int transB)
{
    /* logical strides: A(i,k) = A[i*ai + k*ak], B(k,j) = B[k*bk + j*bj] */
    i64 ai = transA ? sa1 : sa0, ak = transA ? sa0 : sa1;
    i64 bk = transB ? sb1 : sb0, bj = transB ? sb0 : sb1;
    if (M <= 0 || N <= 0) return;
    for (i64 t = 0; t < M * N; t++) C[t] = 0.0f;
    if (K <= 0) return;

    /* Pack B once into [K][N] contiguous so the inner loop vectorises. */
    const float *Bp = B;
    float *Bpack = NULL;
    if (!(bj == 1 && bk == N)) {
        Bpack = (float *)malloc(sizeof(float) * (size_t)K * (size_t)N);
#pragma omp parallel for schedule(static)
        for (i64 k = 0; k < K; k++)
            for (i64 j = 0; j < N; j++) Bpack[k * N + j] = B[k * bk + j * bj];
        Bp = Bpack;
    }
    i64 nIB = (M + MM_IT - 1) / MM_IT;
    i64 nJB = (N + MM_JT - 1) / MM_JT;
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
    for (i64 jb = 0; jb < nJB; jb++)
        for (i64 ib = 0; ib < nIB; ib++) {
            i64 i0 = ib * MM_IT, j0 = jb * MM_JT;
            i64 ni = M - i0 < MM_IT ? M - i0 : MM_IT;
            i64 nj = N - j0 < MM_JT ? N - j0 : MM_JT;
            float acc[MM_IT][MM_JT];
            for (i64 di = 0; di < MM_IT; di++)
                for (i64 dj = 0; dj < MM_JT; dj++) acc[di][dj] = 0.0f;
            if (ni == MM_IT && nj == MM_JT) {
                for (i64 k = 0; k < K; k++) {
                    const float *brow = Bp + k * N + j0;
                    float a0 = A[(i0 + 0) * ai + k * ak], a1 = A[(i0 + 1) * ai + k * ak];
                    float a2 = A[(i0 + 2) * ai + k * ak], a3 = A[(i0 + 3) * ai + k * ak];
#pragma omp simd
                    for (int dj = 0; dj < MM_JT; dj++) {
                        float b = brow[dj];
                        acc[0][dj] = fmaf(a0, b, acc[0][dj]);
                        acc[1][dj] = fmaf(a1, b, acc[1][dj]);
                        acc[2][dj] = fmaf(a2, b, acc[2][dj]);
                        acc[3][dj] = fmaf(a3, b, acc[3][dj]);
                    }
                }
            } else {
                for (i64 k = 0; k < K; k++)
                    for (i64 di = 0; di < ni; di++) {
                        float a = A[(i0 + di) * ai + k * ak];
                        for (i64 dj = 0; dj < nj; dj++)
                            acc[di][dj] = fmaf(a, Bp[k * N + j0 + dj], acc[di][dj]);
                    }
            }
            for (i64 di = 0; di < ni; di++)
                for (i64 dj = 0; dj < nj; dj++) C[(i0 + di) * N + j0 + dj] = acc[di][dj];
        }
    free(Bpack);
}

/* ------------------------------------------------------------------------- *
 * conv2d -- backend/cpu/convolution.cpp:12-52
 *   O[n][oc][oh][ow] = fold over (i in ICg, kh, kw) ascending of
 *   fmaf(I[n][g*ICg+i][h][w], K[oc][i][kh][kw], .), taps outside the image
 *   SKIPPED (convolution.cpp:38-39,43-44), OH = (H+2p-KH)/s+1 (:17-18).
 *   NCHW input, [OC][IC/groups][KH][KW] kernel, both contiguous.
 * ------------------------------------------------------------------------- */
void oracle_conv2d(const float *I, const float *Kw, float *O, i64 N, i64 IC, i64 H, i64 W,
                   i64 OC, i64 KH, i64 KW, i64 sH, i64 sW, i64 pH, i64 pW, i64 groups)
{
    i64 OH = (H + 2 * pH - KH) / sH + 1, OW = (W + 2 * pW - KW) / sW + 1;
    i64 ICg = IC / groups, OCg = OC / groups;
#pragma omp parallel for collapse(3) schedule(static)
    for (i64 n = 0; n < N; n++)
        for (i64 oc = 0; oc < OC; oc++)
            for (i64 oh = 0; oh < OH; oh++) {
                i64 g = oc / OCg;
                for (i64 ow = 0; ow < OW; ow++) {
                    float sum = 0.0f;
                    for (i64 i = 0; i < ICg; i++) {
                        i64 ic = g * ICg + i;
                        for (i64 kh = 0; kh < KH; kh++) {
                            i64 h = oh * sH - pH + kh;
                            if (h < 0 || h >= H) continue;
                            for (i64 kw = 0; kw < KW; kw++) {
                                i64 w = ow * sW - pW + kw;
                                if (w < 0 || w >= W) continue;
                                sum = fmaf(I[((n * IC + ic) * H + h) * W + w],
                                           Kw[((oc * ICg + i) * KH + kh) * KW + kw], sum);
                            }
                        }
                    }
                    O[((n * OC + oc) * OH + oh) * OW + ow] = sum;
                }
            }
}

/* conv2d_grad_input -- backend/cpu/convolution.cpp:54-90
 *   GI[n][ic][h][w] = fold over (oc, kh, kw) ascending of
 *   fmaf(GO[n][oc][oh][ow], K[oc][ic][kh][kw], .) with oh = (h-kh+p)/s kept only
 *   when it divides exactly and lies in [0,OH) (:75-82).  C integer division
 *   truncates toward zero, so a negative numerator with |num| < s gives oh = 0
 *   with a non-zero remainder and is skipped by the remainder test, exactly as
 *   in the reference.  No groups. */
void oracle_conv2d_grad_input(const float *GO, const float *Kw, float *GI, i64 N, i64 IC, i64 H,
                              i64 W, i64 OC, i64 KH, i64 KW, i64 OH, i64 OW, i64 sH, i64 sW,
                              i64 pH, i64 pW)
{
#pragma omp parallel for collapse(3) schedule(static)
    for (i64 n = 0; n < N; n++)
        for (i64 ic = 0; ic < IC; ic++)
            for (i64 h = 0; h < H; h++)
                for (i64 w = 0; w < W; w++) {
                    float sum = 0.0f;
                    for (i64 oc = 0; oc < OC; oc++)
                        for (i64 kh = 0; kh < KH; kh++) {
                            i64 nh = h - kh + pH;
                            i64 oh = nh / sH;
                            if (oh < 0 || oh >= OH || (nh % sH)) continue;
                            for (i64 kw = 0; kw < KW; kw++) {
                                i64 nw = w - kw + pW;
                                i64 ow = nw / sW;
                                if (ow < 0 || ow >= OW || (nw % sW)) continue;
                                sum = fmaf(GO[((n * OC + oc) * OH + oh) * OW + ow],
                                           Kw[((oc * IC + ic) * KH + kh) * KW + kw], sum);
                            }
                        }
                    GI[((n * IC + ic) * H + h) * W + w] = sum;
                }
}

/* conv2d_grad_kernel -- backend/cpu/convolution.cpp:92-128
 *   GK[oc][ic][kh][kw] = fold over (n, oh, ow) ascending, skipping taps outside
 *   the image, of fmaf(GO[n][oc][oh][ow], I[n][ic][h][w], .).  No groups. */
void oracle_conv2d_grad_kernel(const float *GO, const float *I, float *GK, i64 N, i64 IC, i64 H,
                               i64 W, i64 OC, i64 KH, i64 KW, i64 OH, i64 OW, i64 sH, i64 sW,
                               i64 pH, i64 pW)
{
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (i64 oc = 0; oc < OC; oc++)
        for (i64 ic = 0; ic < IC; ic++)
            for (i64 kh = 0; kh < KH; kh++)
                for (i64 kw = 0; kw < KW; kw++) {
                    float sum = 0.0f;
                    for (i64 n = 0; n < N; n++)
                        for (i64 oh = 0; oh < OH; oh++) {
                            i64 h = oh * sH - pH + kh;
                            if (h < 0 || h >= H) continue;
                            for (i64 ow = 0; ow < OW; ow++) {
                                i64 w = ow * sW - pW + kw;
                                if (w < 0 || w >= W) continue;
                                sum = fmaf(GO[((n * OC + oc) * OH + oh) * OW + ow],
                                           I[((n * IC + ic) * H + h) * W + w], sum);
                            }
                        }
                    GK[((oc * IC + ic) * KH + kh) * KW + kw] = sum;
                }
}

/* ------------------------------------------------------------------------- *
 * Fixed-order sums -- backend/cpu/summation.cpp
 *   Every sum is a strict left-to-right fp32 chain from +0, multiplied once at
 *   the end by factor = float(average ? 1.0/count : 1.0) (a double division
 *   rounded to fp32 by the assignment, summation.cpp:15,26,45,63).
 * ------------------------------------------------------------------------- */
static float mean_factor(int average, i64 count)
{
    return average ? (float)(1.0 / (double)count) : 1.0f;
}

/* sum1d -- summation.cpp:12-20.  One chain; `volatile`-free but must not be
 * vectorised: -ffp-contract=off and no -ffast-math keep the order. */
float oracle_sum1d(const float *x, i64 n, int average)
{
    float sum = 0.0f;
    for (i64 i = 0; i < n; i++) sum += x[i];
    return mean_factor(average, n) * sum;
}

/* Chain continued from a given state: lets tests walk 2^30 elements in pieces
 * (sum1d's loop body, summation.cpp:17-18, with the accumulator carried over). */
float oracle_sum1d_carry(const float *x, i64 n, float carry)
{
    float sum = carry;
    for (i64 i = 0; i < n; i++) sum += x[i];
    return sum;
}

/* sum2d_dim0 -- summation.cpp:22-39: per column j, chain over rows. */
void oracle_sum2d_dim0(const float *x, float *out, i64 M, i64 N, int average)
{
    float factor = mean_factor(average, M);
    for (i64 j = 0; j < N; j++) out[j] = 0.0f;
    /* row-major walk: out[j] receives rows in ascending order = same chains */
    for (i64 i = 0; i < M; i++)
        for (i64 j = 0; j < N; j++) out[j] += x[i * N + j];
    for (i64 j = 0; j < N; j++) out[j] = factor * out[j];
}

/* sum2d_dim1 -- summation.cpp:41-58: per row i, chain over columns. */
void oracle_sum2d_dim1(const float *x, float *out, i64 M, i64 N, int average)
{
    float factor = mean_factor(average, N);
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < M; i++) {
        float sum = 0.0f;
        for (i64 j = 0; j < N; j++) sum += x[i * N + j];
        out[i] = factor * sum;
    }
}

/* sum4d_dim023 -- summation.cpp:59-78: per channel c, chain over (n, h, w). */
void oracle_sum4d_dim023(const float *x, float *out, i64 N, i64 C, i64 H, i64 W, int average)
{
    float factor = mean_factor(average, N * H * W);
#pragma omp parallel for schedule(static)
    for (i64 c = 0; c < C; c++) {
        float sum = 0.0f;
        for (i64 n = 0; n < N; n++)
            for (i64 t = 0; t < H * W; t++) sum += x[(n * C + c) * H * W + t];
        out[c] = factor * sum;
    }
}

/* ------------------------------------------------------------------------- *
 * Elementwise math
 * ------------------------------------------------------------------------- */

/* exp2d -- backend/cpu/math.cpp:14-30: (float)exp((double)x) with the system
 * libm.  This is a double rounding (exact -> fp64 by libm -> fp32 by the cast);
 * it is NOT always the correctly rounded fp32 exp. */
void oracle_exp(const float *x, float *y, i64 n)
{
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < n; i++) y[i] = (float)exp((double)x[i]);
}

/* log1d -- backend/cpu/math.cpp:32-47: (float)log((double)x). */
void oracle_log(const float *x, float *y, i64 n)
{
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < n; i++) y[i] = (float)log((double)x[i]);
}

/* div -- repdl/ops.py:98-103: ATen's IEEE fp32 division.  NaN rule of the x86
 * divss/vdivps ATen compiles to: if the dividend is NaN it is returned quieted,
 * else if the divisor is NaN that one is; invalid (0/0, inf/inf) gives the
 * default NaN 0xFFC00000. */
void oracle_div(const float *x, const float *d, float *y, i64 n, int scalar_divisor)
{
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < n; i++) y[i] = x[i] / d[scalar_divisor ? 0 : i];
}

/* sqrt -- repdl/ops.py:122-123: fp32 -> fp64, ATen sqrt, -> fp32.  Rounding a
 * correctly rounded fp64 square root of an fp32 value to fp32 equals the
 * correctly rounded fp32 square root (53 >= 2*24+2).  NaN inputs come back
 * quieted with sign and payload kept; a negative input gives the POSITIVE
 * default NaN 0x7FC00000 in torch 2.11's vectorised CPU kernel (observed; the
 * scalar sqrtsd would give 0xFFC00000), which is what is restated here. */
void oracle_sqrt(const float *x, float *y, i64 n)
{
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < n; i++) {
        float v = x[i];
        if (v != v)
            y[i] = u2f(f2u(v) | 0x00400000u);
        else if (v < 0.0f)
            y[i] = u2f(0x7FC00000u);
        else
            y[i] = (float)sqrt((double)v);
    }
}

/* Row maximum as ATen's max(dim) computes it for the composites below
 * (softmax.cpp:17, cross_entropy.cpp:17): NaN-propagating. */
static float row_max(const float *row, i64 n)
{
    float m = row[0];
    for (i64 j = 1; j < n; j++) {
        float v = row[j];
        if (v != v) { if (m == m) m = v; }
        else if (m == m && v > m) m = v;
    }
    return m;
}

/* softmax -- backend/cpu/softmax.cpp:15-21
 *   e = exp2d(x - rowmax(x)); e /= sum2d_dim1(e) (IEEE division). */
void oracle_softmax(const float *x, float *y, i64 M, i64 N)
{
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < M; i++) {
        const float *row = x + i * N;
        float m = row_max(row, N);
        float sum = 0.0f;
        for (i64 j = 0; j < N; j++) {
            float e = (float)exp((double)(row[j] - m));
            y[i * N + j] = e;
            sum += e;
        }
        for (i64 j = 0; j < N; j++) y[i * N + j] = y[i * N + j] / sum;
    }
}

/* cross_entropy -- backend/cpu/cross_entropy.cpp:15-24
 *   z = x - rowmax; l_i = log1d(sum2d_dim1(exp2d(z)))_i - z[i][target_i];
 *   result = sum1d(l, average=true). */
float oracle_cross_entropy(const float *x, const i64 *target, i64 M, i64 N, float *per_row)
{
    float *l = per_row ? per_row : (float *)malloc(sizeof(float) * (size_t)M);
    for (i64 i = 0; i < M; i++) {
        const float *row = x + i * N;
        float m = row_max(row, N);
        float sum = 0.0f;
        for (i64 j = 0; j < N; j++) sum += (float)exp((double)(row[j] - m));
        float lg = (float)log((double)sum);
        l[i] = lg - (row[target[i]] - m);
    }
    float r = oracle_sum1d(l, M, 1);
    if (!per_row) free(l);
    return r;
}

/* ---- optimizer steps -------------------------------------------------------------------------
 * Adam.step, repdl/optim.py:56-83, element by element in the order of the tensor operations there:
 *   :67-68 grad.add(param, alpha=wd)            -> ATen add with alpha: one fused multiply-add
 *   :70    exp_avg.mul_(b1).add_(grad, alpha=1-b1) -> a multiply, then one fused multiply-add
 *   :71    exp_avg_sq.mul_(b2).add_(mul(grad, grad).mul(1-b2)) -> four separately rounded ops
 *   :73-76 maximum (amsgrad), :77-82 div(sqrt(.), sqrt(bc2)).add_(eps), :83-84 the update.
 * Python scalars reach the fp32 kernels converted to fp32; the callers pass them converted.
 * vmax may be NULL (no amsgrad). */
void oracle_adam_step(float *p, const float *g, float *m, float *v, float *vmax, i64 n, float beta1,
                      float one_minus_beta1, float beta2, float one_minus_beta2, float sqrt_bc2,
                      float eps, float neg_step_size, float weight_decay)
{
    for (i64 i = 0; i < n; i++) {
        float gi = g[i];
        if (weight_decay != 0.0f) gi = fmaf(p[i], weight_decay, gi);
        const float mi = fmaf(gi, one_minus_beta1, m[i] * beta1);
        const float gg = gi * gi;
        const float vi = v[i] * beta2 + gg * one_minus_beta2;
        m[i] = mi;
        v[i] = vi;
        float root = vi;
        if (vmax) {
            const float old = vmax[i];
            root = (old != old) ? old : ((vi != vi) ? vi : (old > vi ? old : vi));
            vmax[i] = root;
        }
        float sq;
        oracle_sqrt(&root, &sq, 1);
        const float denom = sq / sqrt_bc2 + eps;
        const float upd = (mi / denom) * neg_step_size;
        p[i] = p[i] + upd;
    }
}

/* p <- p + (g * -lr): two separately rounded operations (the update style of repdl/optim.py:83;
 * the reference has no SGD of its own). */
void oracle_sgd_step(float *p, const float *g, i64 n, float neg_lr)
{
    for (i64 i = 0; i < n; i++) {
        const float t = g[i] * neg_lr;
        p[i] = p[i] + t;
    }
}
