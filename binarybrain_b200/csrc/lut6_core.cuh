// Device-side core of the 6-input stochastic LUT: the 63-node multilinear tree, its reverse
// pass, and the warp-level reduction of the 64 per-table-entry gradients.
//
// A LUT6 node computes  y = sum_{i<64} W[i] * prod_{j<6} (bit_j(i) ? x_j : 1 - x_j)
// (BinaryBrain include/bb/StochasticOperation.h:95-114).  Written as a binary tree of linear interpolations, one
// level per input, a node is  a (1 - x) + b x  =  (a + b)/2 + (x - 1/2) (b - a).  Pushing that rewrite down to the table
// turns the multilinear form into a polynomial in the centred inputs u_j = x_j - 1/2,
//     y = sum_S c[S] prod_{j in S} u_j,
// whose 64 coefficients come from the table by one butterfly per input, (a, b) -> ((a + b)/2, b - a).  In that basis a
// tree node is ONE fma (a + u * b) instead of a subtract and an fma: 63 operations per value instead of 94, same walk,
// same registers:
//     level 1: t1[k] = c[2k] + u0 * c[2k+1]                      k < 32
//     level 2: t2[k] = t1[2k] + u1 * t1[2k+1]                    k < 16   ... down to y at level 6.
// The centred form is also the well-conditioned one: every |u_j| <= 1/2 balances the factor 2 a difference can gain per
// level, and the table gradients come back from the coefficient gradients without the 64-fold cancellation the
// uncentred polynomial (in x_j) would have.
// The reverse pass walks the same tree: the gradient g arriving at a node a + u * b goes on to a unchanged and to b as
// g * u, and adds g * b to that level's input gradient; the 64 gradients that reach level 1 are the coefficient
// gradients, summed over frames and only then mapped back to table-entry gradients by the adjoint butterfly.
//
// Work mapping used by every LUT kernel: one warp owns one output node for a run of frames; in one
// iteration a warp covers 128 frames and lane l handles frames  base + 32*q + l,  q = 0..3, so every
// global access of a warp is one fully used 128-byte line and a bit-packed row needs exactly one
// 32-bit word per q.  Nothing here needs alignment beyond 4 bytes, and frame tails are masked.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace bb200 {

constexpr int kWarpsPerCta   = 8;     // one output node per warp
constexpr int kFramesPerIter = 128;   // 32 lanes x 4 frames
constexpr unsigned kFull     = 0xffffffffu;

// Table -> polynomial coefficients, done by a whole warp: lane l passes table entries 2l and 2l + 1 and gets
// coefficients 2l and 2l + 1 back (input 0 inside the lane, inputs 1..5 across lanes).
__device__ __forceinline__ float2 table_to_coeffs(float2 v, int lane)
{
    v = make_float2(0.5f * (v.x + v.y), v.y - v.x);
#pragma unroll
    for (int b = 0; b < 5; ++b) {
        const float tx = __shfl_xor_sync(kFull, v.x, 1 << b);
        const float ty = __shfl_xor_sync(kFull, v.y, 1 << b);
        const bool upper = (lane >> b) & 1;
        v.x = upper ? v.x - tx : 0.5f * (v.x + tx);
        v.y = upper ? v.y - ty : 0.5f * (v.y + ty);
    }
    return v;
}

// The adjoint map: gradients of the coefficients -> gradients of the table entries (same lane layout).
// For one butterfly (a, b) -> (m, d) = ((a + b)/2, b - a):  da = dm/2 - dd,  db = dm/2 + dd.
__device__ __forceinline__ float2 coeff_grads_to_table(float2 g, int lane)
{
    g = make_float2(0.5f * g.x - g.y, 0.5f * g.x + g.y);
#pragma unroll
    for (int b = 0; b < 5; ++b) {
        const float tx = __shfl_xor_sync(kFull, g.x, 1 << b);
        const float ty = __shfl_xor_sync(kFull, g.y, 1 << b);
        const bool upper = (lane >> b) & 1;                  // the upper lane holds dd and receives dm, the lower one the reverse
        g.x = upper ? fmaf(0.5f, tx, g.x) : fmaf(0.5f, g.x, -tx);
        g.y = upper ? fmaf(0.5f, ty, g.y) : fmaf(0.5f, g.y, -ty);
    }
    return g;
}

// Input conditioning of the reference's CPU path (include/bb/DifferentiableLutN.h:779-786), returning the centred
// input u = x - 1/2: binary mode maps x to 0.5 +/- bias by (x > 0.5), otherwise x is clipped to [0, 1].
__device__ __forceinline__ float condition_u(float v, int binary, float bias)
{
    return binary ? (v > 0.5f ? bias : -bias) : __saturatef(v) - 0.5f;
}

// Sums acc[i] over the 32 lanes of a warp with a halving butterfly (62 shuffles instead of 64 x 5):
// afterwards lane l holds the warp totals of entries 2l and 2l+1 in acc[0], acc[1].
template <int N, int MASK>
__device__ __forceinline__ void butterfly_step(float (&a)[64], int lane)
{
    const bool upper = (lane & MASK) != 0;
#pragma unroll
    for (int i = 0; i < N / 2; ++i) {
        float send = upper ? a[i] : a[i + N / 2];
        float keep = upper ? a[i + N / 2] : a[i];
        a[i] = keep + __shfl_xor_sync(kFull, send, MASK);
    }
}

__device__ __forceinline__ void warp_reduce_scatter64(float (&a)[64], int lane)
{
    butterfly_step<64, 16>(a, lane);
    butterfly_step<32, 8>(a, lane);
    butterfly_step<16, 4>(a, lane);
    butterfly_step<8, 2>(a, lane);
    butterfly_step<4, 1>(a, lane);
}

__device__ __forceinline__ double warp_sum(double v)
{
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(kFull, v, m);
    return v;
}

}   // namespace bb200

// ---------------------------------------------------------------------------------------------------
// Packed-pair arithmetic (sm_100 f32x2): one instruction does the same fp32 operation on two frames held in a
// 64-bit register pair, so the 63-node tree of two frames costs 63 issue slots instead of 126.  Each lane carries
// NP pairs; the tree is walked depth first (a node's value is produced and consumed before its sibling subtree is
// started), which keeps about one live value per level and pair instead of 32.
// ---------------------------------------------------------------------------------------------------
namespace bb200 {

typedef unsigned long long f32x2;

__device__ __forceinline__ f32x2 pack2(float a, float b) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ void unpack2(f32x2 v, float &a, float &b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) { f32x2 d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) { f32x2 d; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) { f32x2 d; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) { f32x2 d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }

// Per-node table for the packed path: 32 entries of (c0, c0, c1, c1), the coefficient pair of a level-1 node duplicated for
// both halves of a packed operand, so that level 1 reads both operands with one 128-bit load.
__device__ __forceinline__ void stage_table_x2(float4 *tab, const float *__restrict__ W, int node, int lane, int lut_binarize)
{
    __syncwarp();
    float2 v = reinterpret_cast<const float2 *>(W + (size_t)node * 64)[lane];
    if (lut_binarize) {
        v.x = v.x > 0.5f ? 1.0f : 0.0f;
        v.y = v.y > 0.5f ? 1.0f : 0.0f;
    }
    v = table_to_coeffs(v, lane);
    tab[lane] = make_float4(v.x, v.x, v.y, v.y);
    __syncwarp();
}

template <int L, int K, int NP>
struct PolyTree {
    // value of node K at level L for NP frame pairs; x[j][p] is input j of pair p
    static __device__ __forceinline__ void eval(const float4 *tab, const f32x2 (&x)[6][NP], f32x2 (&out)[NP])
    {
        f32x2 a[NP], b[NP];
        PolyTree<L - 1, 2 * K, NP>::eval(tab, x, a);
        PolyTree<L - 1, 2 * K + 1, NP>::eval(tab, x, b);
#pragma unroll
        for (int p = 0; p < NP; ++p) out[p] = fma2(x[L - 1][p], b[p], a[p]);
    }
};

template <int K, int NP>
struct PolyTree<1, K, NP> {
    static __device__ __forceinline__ void eval(const float4 *tab, const f32x2 (&x)[6][NP], f32x2 (&out)[NP])
    {
        const ulonglong2 wd = *reinterpret_cast<const ulonglong2 *>(tab + K);     // .x = (c0, c0), .y = (c1, c1)
#pragma unroll
        for (int p = 0; p < NP; ++p) out[p] = fma2(x[0][p], wd.y, wd.x);
    }
};

template <int NP>
__device__ __forceinline__ void lut6_forward_x2(const float4 *tab, const f32x2 (&x)[6][NP], f32x2 (&y)[NP])
{
    PolyTree<6, 0, NP>::eval(tab, x, y);
}

// ---------------------------------------------------------------------------------------------------
// One frame, both halves of the tree at once.  The coefficients with input 5 clear (c[0..31]) and set (c[32..63]) form
// two 5-input polynomials in the same variables u0..u4; carried in the two halves of packed operands they cost 31
// packed FMAs together, and y = half0 + u5 * half1.  The reverse pass has the same shape (the gradient of half 1 is
// g * u5), and the 64 accumulators become 32 packed ones: acc2[i] = (dC[i], dC[i + 32]).  This halves the issue slots
// of the backward pass without adding a single live register, unlike packing two FRAMES, which doubles the kept state.
// The arithmetic per half is that of the frame-pair walk (PolyTree), operation for operation, so the forward and the backward
// kernels see bit-identical LUT values.
// ---------------------------------------------------------------------------------------------------

// Table for this form: 16 entries of (c[2k], c[2k+32], c[2k+1], c[2k+33]).
__device__ __forceinline__ void stage_table_halves(float4 *tab2, const float *__restrict__ W, int node, int lane, int lut_binarize)
{
    __syncwarp();
    float2 v = reinterpret_cast<const float2 *>(W + (size_t)node * 64)[lane];
    if (lut_binarize) {
        v.x = v.x > 0.5f ? 1.0f : 0.0f;
        v.y = v.y > 0.5f ? 1.0f : 0.0f;
    }
    v = table_to_coeffs(v, lane);
    const float hx = __shfl_down_sync(kFull, v.x, 16), hy = __shfl_down_sync(kFull, v.y, 16);
    if (lane < 16) tab2[lane] = make_float4(v.x, hx, v.y, hy);
    __syncwarp();
}

// The odd operands of levels 2..5 (both halves) and of level 6, kept between the forward and the reverse pass.
struct KeptHalves {
    f32x2 d2[8], d3[4], d4[2], d5;
    float d6;
};

__device__ __forceinline__ float lut6_forward_keep_halves(const float4 *tab2, const float (&u)[6], KeptHalves &D)
{
    f32x2 U[5];
#pragma unroll
    for (int j = 0; j < 5; ++j) U[j] = pack2(u[j], u[j]);
    f32x2 t[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        const ulonglong2 c = *reinterpret_cast<const ulonglong2 *>(tab2 + k);       // .x = even pair, .y = odd pair
        t[k] = fma2(U[0], c.y, c.x);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) { D.d2[k] = t[2 * k + 1]; t[k] = fma2(U[1], D.d2[k], t[2 * k]); }
#pragma unroll
    for (int k = 0; k < 4; ++k) { D.d3[k] = t[2 * k + 1]; t[k] = fma2(U[2], D.d3[k], t[2 * k]); }
#pragma unroll
    for (int k = 0; k < 2; ++k) { D.d4[k] = t[2 * k + 1]; t[k] = fma2(U[3], D.d4[k], t[2 * k]); }
    D.d5 = t[1];
    const f32x2 top = fma2(U[4], D.d5, t[0]);
    float a, b;
    unpack2(top, a, b);
    D.d6 = b;
    return fmaf(u[5], b, a);
}

// Forward only (no kept operands): 31 packed FMAs and one scalar.
__device__ __forceinline__ float lut6_forward_halves(const float4 *tab2, const float (&u)[6])
{
    f32x2 t[16];
    {
        const f32x2 U0 = pack2(u[0], u[0]);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const ulonglong2 c = *reinterpret_cast<const ulonglong2 *>(tab2 + k);
            t[k] = fma2(U0, c.y, c.x);
        }
    }
#pragma unroll
    for (int L = 1; L < 5; ++L) {
        const f32x2 U = pack2(u[L], u[L]);
#pragma unroll
        for (int k = 0; k < (16 >> L); ++k) t[k] = fma2(U, t[2 * k + 1], t[2 * k]);
    }
    float a, b;
    unpack2(t[0], a, b);
    return fmaf(u[5], b, a);
}

// Reverse pass for one frame; acc2[i] collects (dC[i], dC[i + 32]).
__device__ __forceinline__ void lut6_reverse_halves(const float4 *tab2, const float (&u)[6], const KeptHalves &D, float g,
                                                    f32x2 (&acc2)[32], float (&dx)[6])
{
    f32x2 U[5];
#pragma unroll
    for (int j = 0; j < 5; ++j) U[j] = pack2(u[j], u[j]);
    f32x2 gt[16], s[5];
    dx[5] = g * D.d6;
    gt[0] = pack2(g, g * u[5]);

    s[4] = mul2(gt[0], D.d5);
    gt[1] = mul2(gt[0], U[4]);

    s[3] = fma2(gt[1], D.d4[1], mul2(gt[0], D.d4[0]));
#pragma unroll
    for (int k = 1; k >= 0; --k) { gt[2 * k + 1] = mul2(gt[k], U[3]); gt[2 * k] = gt[k]; }

    {
        f32x2 a = mul2(gt[0], D.d3[0]), b = mul2(gt[1], D.d3[1]);
        a = fma2(gt[2], D.d3[2], a);
        b = fma2(gt[3], D.d3[3], b);
        s[2] = add2(a, b);
    }
#pragma unroll
    for (int k = 3; k >= 0; --k) { gt[2 * k + 1] = mul2(gt[k], U[2]); gt[2 * k] = gt[k]; }

    {
        f32x2 a = mul2(gt[0], D.d2[0]), b = mul2(gt[1], D.d2[1]);
#pragma unroll
        for (int k = 2; k < 8; k += 2) { a = fma2(gt[k], D.d2[k], a); b = fma2(gt[k + 1], D.d2[k + 1], b); }
        s[1] = add2(a, b);
    }
#pragma unroll
    for (int k = 7; k >= 0; --k) { gt[2 * k + 1] = mul2(gt[k], U[1]); gt[2 * k] = gt[k]; }

    {
        f32x2 a = 0ull, b = 0ull;
#pragma unroll
        for (int k = 0; k < 16; k += 2) {
            a = fma2(gt[k], reinterpret_cast<const ulonglong2 *>(tab2 + k)->y, a);
            b = fma2(gt[k + 1], reinterpret_cast<const ulonglong2 *>(tab2 + k + 1)->y, b);
        }
        s[0] = add2(a, b);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            acc2[2 * k]     = add2(acc2[2 * k], gt[k]);
            acc2[2 * k + 1] = fma2(gt[k], U[0], acc2[2 * k + 1]);
        }
    }
#pragma unroll
    for (int j = 0; j < 5; ++j) {
        float lo, hi;
        unpack2(s[j], lo, hi);
        dx[j] = lo + hi;
    }
}

}   // namespace bb200
