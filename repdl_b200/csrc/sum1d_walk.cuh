// The inner loop of sum1d's walker (sum1d.cu): one warp, all lanes doing the same thing, carries the
// exact fp32 state through one staged batch of items.
//
// What the loop pays for is the number of instructions on its single dependent path (about four
// cycles each) and dependent branches (about 25 cycles each), so:
//   * the staged item (WItem) holds the validity test as ONE unsigned range test on the state's bit
//     pattern, the step to the successor in bytes, and the kind as a field of its own;
//   * the position is a byte offset p into the staged items, which is also the float offset of the
//     item's leaf elements in the staged raw area (32-byte items, 32-float leaves);
//   * the successor its[p + step] is loaded before the test, so an item that applies -- whatever its
//     kind -- takes one branch; K_HARD is recognised before the test (its kind is known early);
//   * the slot after the batch's last item holds an end marker that fails every test, which saves
//     the bounds check; loads past it are clamped, the position itself may overshoot (a composed
//     run whose parts continue in the next batch).
#pragma once

#include "sum1d_core.cuh"

namespace repdl_b200 {
namespace s1 {

constexpr int K_END = 5;  // walker-only kind: end of the staged batch

struct alignas(16) WItem {
    // For a fixed hypothesis (sign and exponent field) the state's bit pattern, read as an unsigned
    // integer, grows with |m|, so "hypothesis matches and lo <= m < hi" is one range test on the
    // bits: valid iff bits - blo < width (unsigned); width 0: nothing to apply.
    unsigned blo, width;
    int d0, delta;  // increment of the bit pattern for even |m|; d1 - d0
    int kind;       // ItemKind or K_END
    int stepb;      // bytes to the successor when the item applies (32 * items)
    int start, len; // in leaves (spans)
};
static_assert(sizeof(WItem) == 32, "the position doubles as the float offset of the leaf's elements");

#if defined(__CUDACC__)
__device__ __forceinline__ WItem witem_end() { return {0u, 0u, 0, 0, K_END, 32, 0, 0}; }

// Item of the stream -> staged form.
__device__ __forceinline__ WItem witem_from(const int4 a, const int4 c)  // d0 d1 lo hi | sek kind_skip start len
{
    const int kind = c.y & 255;
    // m + lo >= 2^23 and m + hi < 2^24, intersected with the binade's own range of m
    const int mlo = max(M_LO - a.z, M_LO), mhi = min(M_HI - a.w, M_HI);
    const bool summarises = kind <= K_LEAF && mhi > mlo;
    return {((unsigned)c.x << 23) + (unsigned)(mlo - M_LO), summarises ? (unsigned)(mhi - mlo) : 0u, a.x,
            a.y - a.x, kind, 32 * (kind == K_SOFT ? 1 + (c.y >> 8) : 1), c.z, c.w};
}

struct WalkCounts {
    int applied, leaves, soft_fail;
};

enum { WALK_END = 0, WALK_SPAN = 1 };

// Walks the staged items from byte offset p (< endp) on; `its` and `raw` are shared-memory
// addresses, its + endp holds the end marker.  Returns WALK_END (p >= endp: the batch is done; p may
// overshoot) or WALK_SPAN (the item at p is a K_RUN that does not fit or a K_RAWSPAN: the caller
// walks its span and goes on behind it).
template <bool COUNT>
__device__ __forceinline__ int walk_batch(const unsigned char *its, const float *raw, int endp, int &p_io,
                                          int &bits_io, WalkCounts &cnt)
{
    int p = p_io, bits = bits_io;
    uint4 c0 = *reinterpret_cast<const uint4 *>(its + p);     // blo width d0 delta
    int2 c1 = *reinterpret_cast<const int2 *>(its + p + 16);  // kind stepb
    int why = WALK_END;
    for (;;) {
        const int np = p + c1.y;
        const int la = min(np, endp);
        const uint4 n0 = *reinterpret_cast<const uint4 *>(its + la);
        const int2 n1 = *reinterpret_cast<const int2 *>(its + la + 16);
        if (c1.x != K_HARD) {  // (known long before the test below: a cheap branch)
            if ((unsigned)bits - c0.x < c0.y) {
                bits += (int)c0.z + ((bits & 1) ? (int)c0.w : 0);  // |m| stays inside [2^23, 2^24)
                p = np, c0 = n0, c1 = n1;
                if (COUNT) cnt.applied++;
                continue;
            }
            if (c1.x == K_SOFT) {  // a composed run that does not fit: on to its parts
                p += 32;
                c0 = *reinterpret_cast<const uint4 *>(its + p);
                c1 = *reinterpret_cast<const int2 *>(its + p + 16);
                cnt.soft_fail++;
                continue;
            }
            if (c1.x != K_LEAF) {
                why = c1.x != K_END ? WALK_SPAN : WALK_END;
                break;
            }
        }
        // real additions: a K_HARD leaf, or a K_LEAF whose summary does not fit
        const float4 *r4 = reinterpret_cast<const float4 *>(raw + p);
        float4 v[LEAF / 4];
#pragma unroll
        for (int k = 0; k < LEAF / 4; k++) v[k] = r4[k];
        float s = __int_as_float(bits);
#pragma unroll
        for (int k = 0; k < LEAF / 4; k++) {
            s = __fadd_rn(s, v[k].x);
            s = __fadd_rn(s, v[k].y);
            s = __fadd_rn(s, v[k].z);
            s = __fadd_rn(s, v[k].w);
        }
        bits = __float_as_int(s);
        cnt.leaves++;
        p = np, c0 = n0, c1 = n1;  // these kinds step by one
    }
    p_io = p, bits_io = bits;
    return why;
}
#endif

}  // namespace s1
}  // namespace repdl_b200
