// Bit-input LUT layers by pattern table.
//
// With bit-packed inputs every input of a node is one of two values (0.5 - bias, 0.5 + bias), so a node's LUT value over a
// frame depends only on the frame's 6-bit input pattern p: y = Y[p], 64 values per node.  Everything a bit-in / bit-out
// layer produces then follows from Y and from how often each pattern occurs:
//
//   * bit output (y > 0.5 after the optional batch-norm affine map) is a 64-bit truth table B[p] per node, and the layer's
//     forward IS a BinaryLut6 forward with that table: 63 word-wide integer operations per 32 frames instead of a 63-node
//     fp32 tree per frame;
//   * the batch statistics of the training forward are  sum_p H[p] Y[p]  and  sum_p H[p] Y[p]^2  with H the per-node
//     histogram of the patterns over the frames (minterm masks and population counts on whole words).
//
// Y[p] is evaluated by the same tree walk, on the same conditioned inputs (+-bias), as the per-frame kernels, so the
// values -- and every threshold decision taken on them -- are bit-identical to evaluating the tree frame by frame.
//
// Reference semantics: the bit-input branches of include/bb/StochasticLutN.h:432-560 and include/bb/DifferentiableLutN.h:
// 747-905 (CPU), operators bbcu_bit_bit_fp32_StochasticLut_Forward, bbcu_bit_fp32_DifferentiableLutN_ForwardTraining /
// _ForwardInference (include/bbcu/bbcu.h:540-560, 600-618, 712-727).
#include <map>
#include <mutex>

#include "common.cuh"
#include "bit_transpose.cuh"
#include "lut6_core.cuh"

namespace bb200 {

namespace {

enum { kTableRaw = 0, kTableNorm = 1, kTableNone = 2 };

// One warp per node: lane l evaluates patterns l and l + 32 as one packed pair (they differ in input 5 only).
// MODE kTableRaw : B[p] = Y[p] > 0.5                                   (StochasticLut6, bit -> bit)
//      kTableNorm: B[p] = ((Y[p] - mean) * scale) * gamma + beta > 0.5 (DifferentiableLut6 inference; scale = 1/sqrt(var))
//      kTableNone: Y only (training: the statistics come first)
template <int MODE>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
k_pattern_values(const float *__restrict__ W, float *__restrict__ Y, int *__restrict__ table, const float *__restrict__ mean_buf,
                 const float *__restrict__ var_buf, float gamma, float beta, float bias, int O, int lut_binarize)
{
    __shared__ float4 s_tab[kWarpsPerCta][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int node = blockIdx.x * kWarpsPerCta + warp;
    if (node >= O) return;
    float4 *tab = s_tab[warp];
    stage_table_x2(tab, W, node, lane, lut_binarize);
    f32x2 up[6][1], yp[1];
#pragma unroll
    for (int j = 0; j < 5; ++j) {
        const float u = ((lane >> j) & 1) ? bias : -bias;
        up[j][0] = pack2(u, u);
    }
    up[5][0] = pack2(-bias, bias);
    lut6_forward_x2<1>(tab, up, yp);
    float lo, hi;
    unpack2(yp[0], lo, hi);
    if (Y != nullptr) {
        Y[(size_t)node * 64 + lane] = lo;
        Y[(size_t)node * 64 + 32 + lane] = hi;
    }
    if (MODE != kTableNone) {
        if (MODE == kTableNorm) {
            const float mean = mean_buf[node], scale = 1.0f / sqrtf(var_buf[node]);       // DifferentiableLutN.h:866-868
            lo = (lo - mean) * scale; lo = lo * gamma + beta;
            hi = (hi - mean) * scale; hi = hi * gamma + beta;
        }
        const unsigned w_lo = __ballot_sync(kFull, lo > 0.5f), w_hi = __ballot_sync(kFull, hi > 0.5f);
        if (lane == 0) { table[2 * (size_t)node] = (int)w_lo; table[2 * (size_t)node + 1] = (int)w_hi; }
    }
}

// Minterm masks of 6 input words, depth first: at the leaves the population counts of the 64 patterns.
template <int L>
struct Minterms {
    static __device__ __forceinline__ void count(uint32_t m, const uint32_t (&x)[6], uint32_t (&cnt)[64], int base)
    {
        Minterms<L - 1>::count(m & ~x[L - 1], x, cnt, base);
        Minterms<L - 1>::count(m & x[L - 1], x, cnt, base + (1 << (L - 1)));
    }
};
template <>
struct Minterms<0> {
    static __device__ __forceinline__ void count(uint32_t m, const uint32_t (&)[6], uint32_t (&cnt)[64], int base) { cnt[base] += __popc(m); }
};

template <int N, int MASK>
__device__ __forceinline__ void butterfly_step_u32(uint32_t (&a)[64], int lane)
{
    const bool upper = (lane & MASK) != 0;
#pragma unroll
    for (int i = 0; i < N / 2; ++i) {
        const uint32_t send = upper ? a[i] : a[i + N / 2];
        const uint32_t keep = upper ? a[i + N / 2] : a[i];
        a[i] = keep + __shfl_xor_sync(kFull, send, MASK);
    }
}

// Per-node histogram of the input patterns.  Warp = one node for a tile of words; each lane takes whole words (32 frames).
__global__ void __launch_bounds__(kWarpsPerCta * 32)
k_pattern_histogram(const uint32_t *__restrict__ x, const int *__restrict__ idx, uint32_t *__restrict__ hist, int O, int F, long long xs, int groups,
                    int tile_words)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / groups;
    const int node = (blockIdx.x % groups) * kWarpsPerCta + warp;
    if (node >= O) return;
    const uint32_t *rows[6];
#pragma unroll
    for (int j = 0; j < 6; ++j) rows[j] = x + (size_t)__ldg(idx + (size_t)node * 6 + j) * xs;
    uint32_t cnt[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) cnt[i] = 0;
    const int words = (F + 31) >> 5;
    const int w_end = min(words, (tile + 1) * tile_words);
    for (int w = tile * tile_words + lane; w < w_end; w += 32) {
        uint32_t xw[6];
#pragma unroll
        for (int j = 0; j < 6; ++j) xw[j] = __ldg(rows[j] + w);
        const int valid = F - w * 32;                                   // frames in this word
        const uint32_t live = valid >= 32 ? 0xffffffffu : ((1u << valid) - 1u);
        Minterms<6>::count(live, xw, cnt, 0);
    }
    butterfly_step_u32<64, 16>(cnt, lane);
    butterfly_step_u32<32, 8>(cnt, lane);
    butterfly_step_u32<16, 4>(cnt, lane);
    butterfly_step_u32<8, 2>(cnt, lane);
    butterfly_step_u32<4, 1>(cnt, lane);
    atomicAdd(hist + (size_t)node * 64 + 2 * lane, cnt[0]);
    atomicAdd(hist + (size_t)node * 64 + 2 * lane + 1, cnt[1]);
}

// Training statistics and the truth table from Y and the histogram (include/bb/DifferentiableLutN.h:804-812 for the statistics).
__global__ void __launch_bounds__(kWarpsPerCta * 32)
k_dl6_bit_train_finalize(const float *__restrict__ Y, const uint32_t *__restrict__ hist, int *__restrict__ table, float *mean_out, float *rstd_out,
                         float *running_mean, float *running_var, float gamma, float beta, float momentum, int O, int F)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int node = blockIdx.x * kWarpsPerCta + warp;
    if (node >= O) return;
    const float y0 = Y[(size_t)node * 64 + lane], y1 = Y[(size_t)node * 64 + 32 + lane];
    const double h0 = (double)hist[(size_t)node * 64 + lane], h1 = (double)hist[(size_t)node * 64 + 32 + lane];
    double s1 = h0 * (double)y0 + h1 * (double)y1;
    double s2 = h0 * ((double)y0 * (double)y0) + h1 * ((double)y1 * (double)y1);
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    const float rF   = 1.0f / (float)F;
    const float mean = (float)s1 * rF;
    const float var  = fmaxf(1.0e-5f, fmaf((float)s2, rF, -(mean * mean)));
    const float rstd = 1.0f / sqrtf(var);
    float lo = (y0 - mean) * rstd, hi = (y1 - mean) * rstd;
    lo = lo * gamma + beta;
    hi = hi * gamma + beta;
    const unsigned w_lo = __ballot_sync(kFull, lo > 0.5f), w_hi = __ballot_sync(kFull, hi > 0.5f);
    if (lane == 0) {
        table[2 * (size_t)node] = (int)w_lo;
        table[2 * (size_t)node + 1] = (int)w_hi;
        running_mean[node] = running_mean[node] * momentum + mean * (1.0f - momentum);
        running_var[node]  = running_var[node]  * momentum + var  * (1.0f - momentum);
        mean_out[node] = mean;
        rstd_out[node] = rstd;
    }
}

// BinaryLut6 leaves the bits past the last frame as its inputs make them; these layers clear them.
__global__ void k_clear_tail_bits(uint32_t *y, int O, int F, long long ys)
{
    const int node = blockIdx.x * blockDim.x + threadIdx.x;
    if (node >= O) return;
    y[(size_t)node * ys + (F >> 5)] &= (1u << (F & 31)) - 1u;
}

// StochasticLut6 bit -> fp32: y[f] = clip(Y[p(f)], 0, 1).  Warp = one node for a tile of words.  Each lane loads one word of each of
// the six rows (32 words per row and step, coalesced); a 32 x 32 bit transpose per row then gives lane l the bits of frame l of
// all 32 words.  The patterns of four consecutive words are assembled at once, one per byte (a four-bit field of every row is
// spread over the bytes by one multiplication), and for each of the 32 words the warp looks its 32 patterns up in the node's 64
// clipped values (shared memory) and stores 32 consecutive frames.
__global__ void __launch_bounds__(kWarpsPerCta * 32)
k_bit_gather_forward(const uint32_t *__restrict__ x, float *__restrict__ y, const int *__restrict__ idx, const float *__restrict__ Y, int O, int F,
                     long long xs, long long ys, int groups, int tile_words)
{
    __shared__ float s_val[kWarpsPerCta][64];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / groups;
    const int node = (blockIdx.x % groups) * kWarpsPerCta + warp;
    if (node >= O) return;
    float *val = s_val[warp];
    val[lane] = __saturatef(Y[(size_t)node * 64 + lane]);
    val[lane + 32] = __saturatef(Y[(size_t)node * 64 + 32 + lane]);
    __syncwarp();
    const uint32_t *rows[6];
#pragma unroll
    for (int j = 0; j < 6; ++j) rows[j] = x + (size_t)__ldg(idx + (size_t)node * 6 + j) * xs;
    const int words = (F + 31) >> 5;
    const int w_end = min(words, (tile + 1) * tile_words);
    float *yrow = y + (size_t)node * ys;
    const BitTranspose transpose(lane);
    for (int w0 = tile * tile_words; w0 < w_end; w0 += 32) {
        uint32_t t[6];
#pragma unroll
        for (int j = 0; j < 6; ++j) t[j] = transpose((w0 + lane < w_end) ? __ldg(rows[j] + w0 + lane) : 0u);      // bit k: frame `lane` of word w0 + k
        const int kn = min(32, w_end - w0);
        float *yw = yrow + (size_t)w0 * 32 + lane;
        const bool whole = kn == 32 && (long long)(w0 + 32) * 32 <= F;         // 32 full words: no guards
#pragma unroll
        for (int k0 = 0; k0 < 32; k0 += 4) {
            if (!whole && k0 >= kn) break;
            uint32_t p4 = 0u;                                                   // the patterns of words k0 .. k0 + 3, one per byte
#pragma unroll
            for (int j = 0; j < 6; ++j) p4 |= ((((t[j] >> k0) & 0xfu) * 0x00204081u) & 0x01010101u) << j;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float v = val[(p4 >> (8 * i)) & 63u];
                if (whole || (k0 + i < kn && (long long)(w0 + k0 + i) * 32 + lane < F)) yw[(k0 + i) * 32] = v;
            }
        }
    }
}

// --------------------------------------------------------------------------------------------- backward of bit-input layers
// With bit inputs the backward pass also factors through the pattern p of a frame:
//   dx_j(f) = g(f) * D_j[p(f)]          D_j[p] = dy/du_j at pattern p, six values per pattern and node
//   dW      = K^T Hg                    Hg[p] = sum of g over the frames with pattern p; K[i][p] = prod_j k(bit_j(i), bit_j(p)),
//                                        k = 0.5 + bias where the bits agree, 0.5 - bias where they differ (one butterfly per input)
// and for the batch-norm form g(f) = mask[p] dy(f) gamma rstd + dmean + Y[p] dvar / F, so Hg and the two batch sums
// (include/bb/DifferentiableLutN.h:1190-1258) follow from Hdy[p] = sum of dy per pattern and the pattern counts H[p].
// Per frame that leaves: the pattern (bit inputs: a 32 x 32 bit transpose per row and 32 words, then four patterns at a time, one per
// byte), 6 table reads, 6 multiplies and the 6 dx reductions.

enum { kBwdPlainAll = 0, kBwdHistOnly = 1, kBwdNormDx = 2 };

struct BitBwdArgs {
    const uint32_t *x;                  // bit-packed rows, or (XF32 kernels) fp32 rows reinterpreted: an input is "set" where x > 0.5
    uint32_t *hist;                     // XF32 only: [O][64] pattern counts (added to by the histogram pass)
    unsigned char *pat;                 // XF32 with batch norm: [O][fs] pattern bytes, written by the histogram pass, read by the dx pass
    const float *dy;
    float *dx;
    const int *idx;
    const float *W;
    float *hdy;                         // [O][64] per-pattern sums of dy (added to)
    const float *mean, *rstd, *dmean, *dvar;
    float gamma, beta, bias, rF;
    int O, F, groups, tile_words, lut_binarize;
    long long xs, fs;                   // word stride of x, float stride of dy / dx
};

// Four CTAs per SM (64 registers): the frame loop needs few registers and hides its load latency with warps; the table set-up at the
// top, which would like ~130, runs once per tile and may spill.
// XF32: the layer is in binary mode on fp32 frames (include/bb/DifferentiableLutN.h:779-786 maps x to 0.5 +- bias by x > 0.5), so the
// pattern of a frame comes from six compares instead of six bits, and the histogram pass also counts the patterns.
template <int MODE, bool XF32>
__global__ void __launch_bounds__(kWarpsPerCta * 32, 4)
k_bit_backward_frames(const BitBwdArgs a)
{
    __shared__ float4 s_tab[kWarpsPerCta][16];
    __shared__ float s_D[kWarpsPerCta][6][64];
    __shared__ float s_A[kWarpsPerCta][64], s_B[kWarpsPerCta][64], s_H[kWarpsPerCta][64];
    __shared__ unsigned s_C[XF32 ? kWarpsPerCta : 1][64];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / a.groups;
    const int node = (blockIdx.x % a.groups) * kWarpsPerCta + warp;
    if (node >= a.O) return;
    // the node's per-pattern tables: this lane works out patterns `lane` and `lane + 32`
    stage_table_halves(s_tab[warp], a.W, node, lane, a.lut_binarize);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int p = lane + 32 * half;
        float u[6];
#pragma unroll
        for (int j = 0; j < 6; ++j) u[j] = ((p >> j) & 1) ? a.bias : -a.bias;
        KeptHalves K;
        const float v = lut6_forward_keep_halves(s_tab[warp], u, K);
        if (MODE != kBwdHistOnly) {
            f32x2 unused[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) unused[i] = 0ull;
            float d[6];
            lut6_reverse_halves(s_tab[warp], u, K, 1.0f, unused, d);
#pragma unroll
            for (int j = 0; j < 6; ++j) s_D[warp][j][p] = d[j];
        }
        if (MODE == kBwdNormDx) {
            const float mean = a.mean[node], rstd = a.rstd[node];
            const float tanh_x = ((v - mean) * rstd) * a.gamma + a.beta;
            s_A[warp][p] = (tanh_x <= 0.0f || tanh_x >= 1.0f) ? 0.0f : 1.0f;              // hard-tanh mask of the pattern
            s_B[warp][p] = a.dmean[node] + (v * a.dvar[node] * a.rF);
        }
        if (MODE != kBwdNormDx) s_H[warp][p] = 0.0f;
        if (XF32 && MODE == kBwdHistOnly) s_C[warp][p] = 0u;
    }
    __syncwarp();
    const float grstd_gamma = a.gamma, rstd_n = (MODE == kBwdNormDx) ? a.rstd[node] : 0.0f;

    const uint32_t *rows[6];
    long long off[6];
#pragma unroll
    for (int j = 0; j < 6; ++j) {
        const int r = __ldg(a.idx + (size_t)node * 6 + j);
        rows[j] = a.x + (size_t)r * a.xs;
        off[j] = (long long)r * a.fs;
    }
    const int words = (a.F + 31) >> 5;
    const int w_end = min(words, (tile + 1) * a.tile_words);
    const float *dyrow = a.dy + (size_t)node * a.fs;
    const BitTranspose transpose(lane);
    for (int w0 = tile * a.tile_words; w0 < w_end; w0 += 32) {
        uint32_t xw[6];                       // bit inputs: after the transpose, bit k of xw[j] is frame `lane` of word w0 + k
        if (!XF32) {
#pragma unroll
            for (int j = 0; j < 6; ++j) xw[j] = transpose((w0 + lane < w_end) ? __ldg(rows[j] + w0 + lane) : 0u);
        }
        uint32_t p4 = 0u;                     // bit inputs: the patterns of four consecutive words, one per byte
        const int kn = min(32, w_end - w0);
        // dy of the next word is fetched while this one is processed
        long long f = (long long)w0 * 32 + lane;
        float dy_next = f < a.F ? __ldg(dyrow + f) : 0.0f;
        // fp32 frames: this step's inputs were fetched during the previous step.  With batch norm the histogram pass leaves one pattern
        // byte per frame behind and the dx pass reads that instead of gathering the six rows a second time.
        constexpr bool kFromBytes = XF32 && MODE == kBwdNormDx;
        float x_next[(XF32 && !kFromBytes) ? 6 : 1];
        unsigned char p_next = 0;
        const unsigned char *prow = XF32 && a.pat != nullptr ? a.pat + (size_t)node * a.fs : nullptr;
        if (kFromBytes) {
            p_next = f < a.F ? prow[f] : (unsigned char)0;
        } else if (XF32) {
#pragma unroll
            for (int j = 0; j < 6; ++j) x_next[j] = f < a.F ? __ldg(reinterpret_cast<const float *>(a.x) + f + off[j]) : 0.0f;
        }
        for (int k = 0; k < kn; ++k, f += 32) {
            uint32_t p = 0;
            if (kFromBytes) {
                p = p_next;
                if (k + 1 < kn && f + 32 < a.F) p_next = prow[f + 32];
            } else if (XF32) {
#pragma unroll
                for (int j = 5; j >= 0; --j) p = (p << 1) | (x_next[j] > 0.5f ? 1u : 0u);
                if (k + 1 < kn && f + 32 < a.F) {
                    const float *xf = reinterpret_cast<const float *>(a.x) + f + 32;
#pragma unroll
                    for (int j = 0; j < 6; ++j) x_next[j] = __ldg(xf + off[j]);
                }
                if (MODE == kBwdHistOnly && f < a.F) const_cast<unsigned char *>(prow)[f] = (unsigned char)p;
            } else {
                if ((k & 3) == 0) {
                    p4 = 0u;
#pragma unroll
                    for (int j = 0; j < 6; ++j) p4 |= ((((xw[j] >> k) & 0xfu) * 0x00204081u) & 0x01010101u) << j;
                }
                p = (p4 >> (8 * (k & 3))) & 63u;
            }
            const float dyv = dy_next;
            if (k + 1 < kn && f + 32 < a.F) dy_next = __ldg(dyrow + f + 32);
            if (f < a.F) {
                if (MODE != kBwdNormDx) atomicAdd(&s_H[warp][p], dyv);
                if (XF32 && MODE == kBwdHistOnly) atomicAdd(&s_C[warp][p], 1u);
                if (MODE != kBwdHistOnly) {
                    float g = dyv;
                    if (MODE == kBwdNormDx) g = ((dyv * s_A[warp][p]) * grstd_gamma) * rstd_n + s_B[warp][p];
                    float *dxf = a.dx + f;
#pragma unroll
                    for (int j = 0; j < 6; ++j) atomicAdd(dxf + off[j], g * s_D[warp][j][p]);
                }
            }
        }
    }
    if (MODE != kBwdNormDx) {
        __syncwarp();
        atomicAdd(a.hdy + (size_t)node * 64 + lane, s_H[warp][lane]);
        atomicAdd(a.hdy + (size_t)node * 64 + 32 + lane, s_H[warp][lane + 32]);
        if (XF32 && MODE == kBwdHistOnly) {
            atomicAdd(a.hist + (size_t)node * 64 + lane, s_C[warp][lane]);
            atomicAdd(a.hist + (size_t)node * 64 + 32 + lane, s_C[warp][lane + 32]);
        }
    }
}

// Per-pattern gradient sums -> table-entry gradients: for every input, (a, b) -> (a hi + b lo, a lo + b hi) with hi = 0.5 + bias,
// lo = 0.5 - bias.  Lane l holds patterns 2l and 2l + 1 on entry and table entries 2l and 2l + 1 on return.
__device__ __forceinline__ float2 pattern_sums_to_table_grads(float2 v, int lane, float bias)
{
    const float hi = 0.5f + bias, lo = 0.5f - bias;
    v = make_float2(v.x * hi + v.y * lo, v.x * lo + v.y * hi);
#pragma unroll
    for (int b = 0; b < 5; ++b) {
        const float tx = __shfl_xor_sync(kFull, v.x, 1 << b), ty = __shfl_xor_sync(kFull, v.y, 1 << b);
        v.x = v.x * hi + tx * lo;
        v.y = v.y * hi + ty * lo;
    }
    return v;
}

// One warp per node.  BN = false: dW += K^T Hdy.  BN = true: the batch sums, dmean / dvar, then dW += K^T Hg with
// Hg[p] = mask[p] gamma rstd Hdy[p] + (dmean + Y[p] dvar / F) H[p].
// `sums_out` (frame-sharded callers): the node's local (dstd, dmeanx) go out as fp64 and nothing else is done.
// `sums_in`: the sums over ALL ranks' frames come in instead of being formed from this rank's Hdy; rF = 1 / total frames.
template <bool BN>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
k_bit_backward_finalize(const float *__restrict__ hdy, const uint32_t *__restrict__ hist, const float *__restrict__ Y, float *dW,
                        const float *__restrict__ mean_buf, const float *__restrict__ rstd_buf, float *dmean_out, float *dvar_out, float gamma,
                        float beta, float bias, int O, float rF, double *sums_out, const double *__restrict__ sums_in)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int node = blockIdx.x * kWarpsPerCta + warp;
    if (node >= O) return;
    float2 hg = reinterpret_cast<const float2 *>(hdy + (size_t)node * 64)[lane];             // patterns 2l, 2l + 1
    if (BN) {
        const float2 y = reinterpret_cast<const float2 *>(Y + (size_t)node * 64)[lane];
        const uint2 h = reinterpret_cast<const uint2 *>(hist + (size_t)node * 64)[lane];
        const float mean = mean_buf[node], rstd = rstd_buf[node], rstd2 = rstd * rstd;
        const float t0 = ((y.x - mean) * rstd) * gamma + beta, t1 = ((y.y - mean) * rstd) * gamma + beta;
        const float m0 = (t0 <= 0.0f || t0 >= 1.0f) ? 0.0f : 1.0f, m1 = (t1 <= 0.0f || t1 >= 1.0f) ? 0.0f : 1.0f;
        const float dxn0 = gamma * (m0 * hg.x), dxn1 = gamma * (m1 * hg.y);                   // sum over the pattern's frames of gamma * masked dy
        double dstd, dmeanx;
        if (sums_in != nullptr) {
            dstd = sums_in[2 * (size_t)node];
            dmeanx = sums_in[2 * (size_t)node + 1];
        } else {
            dstd = -((double)(dxn0 * (y.x - mean) * rstd2) + (double)(dxn1 * (y.y - mean) * rstd2));
            dmeanx = -((double)(dxn0 * rstd) + (double)(dxn1 * rstd));
            dstd = warp_sum(dstd);
            dmeanx = warp_sum(dmeanx);
        }
        if (sums_out != nullptr) {
            if (lane == 0) { sums_out[2 * (size_t)node] = dstd; sums_out[2 * (size_t)node + 1] = dmeanx; }
            return;
        }
        const float dvar = (float)dstd * rstd;
        const float dmean = ((float)dmeanx - (mean * dvar)) * rF;
        if (lane == 0) { dvar_out[node] = dvar; dmean_out[node] = dmean; }
        hg.x = (dxn0 * rstd) + (dmean + (y.x * dvar * rF)) * (float)h.x;
        hg.y = (dxn1 * rstd) + (dmean + (y.y * dvar * rF)) * (float)h.y;
    }
    const float2 gw = pattern_sums_to_table_grads(hg, lane, bias);
    float *dst = dW + (size_t)node * 64 + 2 * lane;
    dst[0] += gw.x;
    dst[1] += gw.y;
}

// --------------------------------------------------------------------------------------------- binary mode on fp32 frames, forward
// Inputs are conditioned to 0.5 +- bias by x > 0.5 (include/bb/DifferentiableLutN.h:779-786), so the same per-pattern values apply;
// the pattern of a frame comes from six compares.  A lane owns four consecutive frames of every 128 (one 128-bit load per input row).
//   PASS_COUNT : pattern counts per node (shared-memory integer atomics, added to `hist` per tile) and the four patterns of the lane
//                as one 32-bit word into `pat` ([node][frame] bytes) for the output pass of the training forward;
//   PASS_OUTPUT: y[f] = val[p(f)], the patterns read back from `pat`;
//   PASS_DIRECT: both in one go, y[f] = val[p(f)] straight from x (StochasticLut6 forward, inference);
//   PASS_STATS : the first half of a frame-sharded training forward: pattern counts, and y[f] = Y[p(f)] unclipped (the raw LUT value the
//                normalise half works on).
// val[p]: clip(Y[p]) (StochasticLut6), or the truth-table bit as 0 / 1 (DifferentiableLut6 in binary mode).
enum { kPassCount = 0, kPassOutput = 1, kPassDirect = 2, kPassStats = 3 };

struct F32BinArgs {
    const float *x;
    float *y;
    const int *idx;
    const float *Y;          // [O][64] per-pattern values (kPassDirect without a table)
    const int *table;        // [O][2] truth tables, or nullptr: val = clip(Y)
    uint32_t *hist;          // [O][64]
    unsigned char *pat;      // [O][fs] pattern bytes
    int O, F, groups, tile_frames;
    long long fs;            // frame stride of x, y and pat (elements); a multiple of 4
};

template <int PASS>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
k_f32_binary_forward(const F32BinArgs a)
{
    __shared__ float    s_val[kWarpsPerCta][64];
    __shared__ unsigned s_cnt[kWarpsPerCta][64];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / a.groups;
    const int node = (blockIdx.x % a.groups) * kWarpsPerCta + warp;
    if (node >= a.O) return;
    constexpr bool kCounts = PASS == kPassCount || PASS == kPassStats;
    if (kCounts) {
        s_cnt[warp][lane] = 0u;
        s_cnt[warp][lane + 32] = 0u;
    }
    if (PASS == kPassStats) {
        s_val[warp][lane] = a.Y[(size_t)node * 64 + lane];
        s_val[warp][lane + 32] = a.Y[(size_t)node * 64 + 32 + lane];
    } else if (PASS == kPassCount) {
    } else if (a.table != nullptr) {
        const uint32_t lo = (uint32_t)a.table[2 * (size_t)node], hi = (uint32_t)a.table[2 * (size_t)node + 1];
        s_val[warp][lane] = ((lo >> lane) & 1u) ? 1.0f : 0.0f;
        s_val[warp][lane + 32] = ((hi >> lane) & 1u) ? 1.0f : 0.0f;
    } else {
        s_val[warp][lane] = __saturatef(a.Y[(size_t)node * 64 + lane]);
        s_val[warp][lane + 32] = __saturatef(a.Y[(size_t)node * 64 + 32 + lane]);
    }
    __syncwarp();
    long long off[6];
    if (PASS != kPassOutput) {
#pragma unroll
        for (int j = 0; j < 6; ++j) off[j] = (long long)__ldg(a.idx + (size_t)node * 6 + j) * a.fs;
    }
    const int f_begin = tile * a.tile_frames, f_end = min(a.F, f_begin + a.tile_frames);
    unsigned char *prow = a.pat ? a.pat + (size_t)node * a.fs : nullptr;
    float *yrow = a.y ? a.y + (size_t)node * a.fs : nullptr;
    // the loads of step i + 1 are issued before step i is processed (the loop body is short and would otherwise wait on every load)
    float4 xq[PASS == kPassOutput ? 1 : 6];
    uint32_t pq = 0;
    auto fetch = [&](int f) {
        if (PASS == kPassOutput) {
            pq = *reinterpret_cast<const uint32_t *>(prow + f);
        } else {
#pragma unroll
            for (int j = 0; j < 6; ++j) xq[j] = __ldg(reinterpret_cast<const float4 *>(a.x + off[j] + f));
        }
    };
    int f = f_begin + 4 * lane;
    if (f < f_end) fetch(f);
    for (; f < f_end; f += 128) {
        uint32_t p4 = pq;                                          // the patterns of frames f .. f+3, one per byte
        if (PASS != kPassOutput) {
            p4 = 0;
#pragma unroll
            for (int j = 0; j < 6; ++j)
                p4 |= ((xq[j].x > 0.5f ? 1u : 0u) | (xq[j].y > 0.5f ? 0x100u : 0u) | (xq[j].z > 0.5f ? 0x10000u : 0u) | (xq[j].w > 0.5f ? 0x1000000u : 0u)) << j;
        }
        if (f + 128 < f_end) fetch(f + 128);
        if (kCounts) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (f + i < a.F) atomicAdd(&s_cnt[warp][(p4 >> (8 * i)) & 63u], 1u);
            if (PASS == kPassCount) *reinterpret_cast<uint32_t *>(prow + f) = p4;
        }
        if (PASS != kPassCount) {
            const float4 o = make_float4(s_val[warp][p4 & 63u], s_val[warp][(p4 >> 8) & 63u], s_val[warp][(p4 >> 16) & 63u], s_val[warp][(p4 >> 24) & 63u]);
            if (f + 3 < a.F) {
                *reinterpret_cast<float4 *>(yrow + f) = o;
            } else {
                const float ov[4] = {o.x, o.y, o.z, o.w};
                for (int i = 0; i < 4 && f + i < a.F; ++i) yrow[f + i] = ov[i];
            }
        }
    }
    if (kCounts) {
        __syncwarp();
        atomicAdd(a.hist + (size_t)node * 64 + lane, s_cnt[warp][lane]);
        atomicAdd(a.hist + (size_t)node * 64 + 32 + lane, s_cnt[warp][lane + 32]);
    }
}

// Per-node (sum y, sum y^2) over this rank's frames from the pattern counts: sums[node] = (sum_p H[p] Y[p], sum_p H[p] Y[p]^2).
__global__ void __launch_bounds__(kWarpsPerCta * 32)
k_counts_to_sums(const float *__restrict__ Y, const uint32_t *__restrict__ hist, double *__restrict__ sums, int O)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int node = blockIdx.x * kWarpsPerCta + warp;
    if (node >= O) return;
    const double y0 = (double)Y[(size_t)node * 64 + lane], y1 = (double)Y[(size_t)node * 64 + 32 + lane];
    const double h0 = (double)hist[(size_t)node * 64 + lane], h1 = (double)hist[(size_t)node * 64 + 32 + lane];
    const double s1 = warp_sum(h0 * y0 + h1 * y1), s2 = warp_sum(h0 * (y0 * y0) + h1 * (y1 * y1));
    if (lane == 0) { sums[2 * (size_t)node] = s1; sums[2 * (size_t)node + 1] = s2; }
}

struct Scratch {
    float    *Y;        // [O][64]
    uint32_t *hist;     // [O][64]
    int      *table;    // [O][2]
    unsigned char *pat; // extra bytes asked for by the caller (pattern bytes of the fp32 binary-mode training forward)
};

// What the statistics half of a frame-sharded backward left in a stream's scratch (pattern counts, per-pattern dy sums, pattern
// bytes), so that the apply half that follows it on the same stream need not repeat that pass.  Any other use of the scratch
// forgets it; the apply half checks every field and redoes the pass when something differs.
struct PassOneRecord {
    const void *x = nullptr, *dy = nullptr, *W = nullptr;
    int O = 0, F = 0;
    long long fs = 0;
};
std::mutex g_record_mu;
std::map<std::pair<int, cudaStream_t>, PassOneRecord> g_records;

std::pair<int, cudaStream_t> record_key(cudaStream_t st)
{
    int dev = 0;
    cudaGetDevice(&dev);
    return std::make_pair(dev, st);
}

bool carve(Scratch &s, int O, cudaStream_t st, size_t extra = 0)
{
    {
        std::lock_guard<std::mutex> g(g_record_mu);
        g_records.erase(record_key(st));
    }
    const size_t per_node = 64 * 4 + 64 * 4 + 8 + 64 * 4;        // Y, pattern counts, truth table, per-pattern dy sums
    const size_t fixed = (per_node * (size_t)O + 255) & ~(size_t)255;
    unsigned char *base = static_cast<unsigned char *>(stream_scratch(st, fixed + extra, 1));
    if (base == nullptr) return false;
    s.pat = base + fixed;
    s.Y = reinterpret_cast<float *>(base);
    s.hist = reinterpret_cast<uint32_t *>(base + (size_t)O * 256);
    s.table = reinterpret_cast<int *>(base + (size_t)O * 768);
    return true;
}

int run_binary_lut(const int *x, int *y, const int *idx, const int *table, int O, int F, int stride, cudaStream_t st)
{
    int rc = bbcu_bit_BinaryLut6_Forward(x, y, idx, table, O, F, stride, reinterpret_cast<bbcu_stream_t>(st));
    if (rc) return rc;
    if (F & 31) {
        k_clear_tail_bits<<<(O + 255) / 256, 256, 0, st>>>(reinterpret_cast<uint32_t *>(y), O, F, stride);
        return launch_status();
    }
    return BBCU_OK;
}

}   // namespace

// StochasticLut6 bit -> bit (with_bn = false) and DifferentiableLut6 bit inference (with_bn = true).  Returns
// BBCU_ERR_NO_MEMORY when the scratch cannot be had; the caller then falls back to the per-frame kernel.
int bit_forward_by_table(bool with_bn, const int *x, int *y, const int *idx, const float *W, const float *rmean, const float *rvar, float gamma,
                         float beta, float bias, int O, int F, int stride, int lut_binarize, cudaStream_t st)
{
    if (O == 0 || F == 0) return BBCU_OK;
    Scratch s;
    if (!carve(s, O, st)) return BBCU_ERR_NO_MEMORY;
    const int blocks = (O + kWarpsPerCta - 1) / kWarpsPerCta;
    if (with_bn) k_pattern_values<kTableNorm><<<blocks, kWarpsPerCta * 32, 0, st>>>(W, nullptr, s.table, rmean, rvar, gamma, beta, bias, O, lut_binarize);
    else         k_pattern_values<kTableRaw><<<blocks, kWarpsPerCta * 32, 0, st>>>(W, nullptr, s.table, nullptr, nullptr, 0.0f, 0.0f, bias, O, lut_binarize);
    BB200_CUDA(cudaPeekAtLastError());
    return run_binary_lut(x, y, idx, s.table, O, F, stride, st);
}

int dl6_bit_forward_training_by_table(const int *x, int *y, const int *idx, const float *W, float *mean, float *rstd, float *rmean, float *rvar,
                                      float gamma, float beta, float momentum, float bias, int O, int F, int stride, int lut_binarize,
                                      cudaStream_t st)
{
    if (O == 0 || F == 0) return BBCU_OK;
    Scratch s;
    if (!carve(s, O, st)) return BBCU_ERR_NO_MEMORY;
    const int groups = (O + kWarpsPerCta - 1) / kWarpsPerCta;
    k_pattern_values<kTableNone><<<groups, kWarpsPerCta * 32, 0, st>>>(W, s.Y, nullptr, nullptr, nullptr, 0.0f, 0.0f, bias, O, lut_binarize);
    BB200_CUDA(cudaPeekAtLastError());
    BB200_CUDA(cudaMemsetAsync(s.hist, 0, (size_t)O * 256, st));
    // word tiles: wide enough to amortise the 64-counter reduction (about 400 instructions per warp), narrow enough to fill the GPU
    const int words = (F + 31) / 32;
    int tile_words = 4096;
    while (tile_words > 32 && (long long)groups * ((words + tile_words - 1) / tile_words) < 2LL * device_info().sm_count) tile_words /= 2;
    const long long blocks = (long long)groups * ((words + tile_words - 1) / tile_words);
    BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
    k_pattern_histogram<<<(unsigned)blocks, kWarpsPerCta * 32, 0, st>>>(reinterpret_cast<const uint32_t *>(x), idx, s.hist, O, F, stride, groups,
                                                                       tile_words);
    BB200_CUDA(cudaPeekAtLastError());
    k_dl6_bit_train_finalize<<<groups, kWarpsPerCta * 32, 0, st>>>(s.Y, s.hist, s.table, mean, rstd, rmean, rvar, gamma, beta, momentum, O, F);
    BB200_CUDA(cudaPeekAtLastError());
    return run_binary_lut(x, y, idx, s.table, O, F, stride, st);
}

// StochasticLut6 bit -> fp32 forward.
int bit_fp32_forward_by_table(const int *x, float *y, const int *idx, const float *W, float bias, int O, int F, long long xs, long long ys,
                              int lut_binarize, cudaStream_t st)
{
    if (O == 0 || F == 0) return BBCU_OK;
    Scratch s;
    if (!carve(s, O, st)) return BBCU_ERR_NO_MEMORY;
    const int groups = (O + kWarpsPerCta - 1) / kWarpsPerCta;
    k_pattern_values<kTableNone><<<groups, kWarpsPerCta * 32, 0, st>>>(W, s.Y, nullptr, nullptr, nullptr, 0.0f, 0.0f, bias, O, lut_binarize);
    BB200_CUDA(cudaPeekAtLastError());
    // frame tiles as in the other LUT kernels: the tile's input rows stay in L2 while all nodes consume them
    const int tf = frame_tile(3LL * O, 1, groups, F, 1 << 20);
    const int tile_words = ((tf + 1023) / 1024) * 32;
    const long long blocks = (long long)groups * (((F + 31) / 32 + tile_words - 1) / tile_words);
    BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
    k_bit_gather_forward<<<(unsigned)blocks, kWarpsPerCta * 32, 0, st>>>(reinterpret_cast<const uint32_t *>(x), y, idx, s.Y, O, F, xs, ys, groups,
                                                                        tile_words);
    return launch_status();
}

// Binary mode on fp32 frames.  mode 0: StochasticLut6 forward (y = clip of the per-pattern value); 1: DifferentiableLut6 inference
// (running statistics); 2: DifferentiableLut6 training forward (batch statistics from the pattern counts); 3: the statistics half of a
// frame-sharded training forward (raw per-pattern values into y, this rank's fp64 sums [O][2] through the `mean` argument).  Declines (NO_MEMORY) when the
// rows are not 16-byte aligned or the pattern bytes of the training forward would not be a reasonable scratch.
int f32_binary_forward_by_table(int mode, const float *x, float *y, const int *idx, const float *W, float *mean, float *rstd, float *rmean,
                                float *rvar, float gamma, float beta, float momentum, float bias, int O, int F, long long fs, int lut_binarize,
                                cudaStream_t st)
{
    if (O == 0 || F == 0) return BBCU_OK;
    if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) != 0 || (fs % 4) != 0) return BBCU_ERR_NO_MEMORY;
    const size_t pat_bytes = mode == 2 ? (size_t)O * (size_t)fs : 0;
    if (pat_bytes > ((size_t)1 << 30)) return BBCU_ERR_NO_MEMORY;
    Scratch s;
    if (!carve(s, O, st, pat_bytes)) return BBCU_ERR_NO_MEMORY;
    F32BinArgs a = {};
    a.x = x; a.y = y; a.idx = idx; a.Y = s.Y; a.hist = s.hist; a.O = O; a.F = F; a.fs = fs;
    a.groups = (O + kWarpsPerCta - 1) / kWarpsPerCta;
    const unsigned threads = kWarpsPerCta * 32;
    // frame tiles narrow enough for the tile's input rows to stay in L2 while every node reads them
    const int tf = frame_tile(3LL * O, 32, a.groups, F, 1 << 20);
    a.tile_frames = ((tf + 127) / 128) * 128;
    if (a.tile_frames < 1024) a.tile_frames = 1024;               // at least eight steps per warp and tile: set-up and the 64 count atomics amortise
    const long long blocks = (long long)a.groups * ((F + a.tile_frames - 1) / a.tile_frames);
    BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
    if (mode == 0) {
        k_pattern_values<kTableNone><<<a.groups, threads, 0, st>>>(W, s.Y, nullptr, nullptr, nullptr, 0.0f, 0.0f, bias, O, lut_binarize);
        BB200_CUDA(cudaPeekAtLastError());
        k_f32_binary_forward<kPassDirect><<<(unsigned)blocks, threads, 0, st>>>(a);
        return launch_status();
    }
    if (mode == 3) {          // first half of a sharded training forward: raw values into y, per-rank sums (mean doubles as the sums pointer)
        k_pattern_values<kTableNone><<<a.groups, threads, 0, st>>>(W, s.Y, nullptr, nullptr, nullptr, 0.0f, 0.0f, bias, O, lut_binarize);
        BB200_CUDA(cudaPeekAtLastError());
        BB200_CUDA(cudaMemsetAsync(s.hist, 0, (size_t)O * 256, st));
        k_f32_binary_forward<kPassStats><<<(unsigned)blocks, threads, 0, st>>>(a);
        BB200_CUDA(cudaPeekAtLastError());
        k_counts_to_sums<<<a.groups, threads, 0, st>>>(s.Y, s.hist, reinterpret_cast<double *>(mean), O);
        return launch_status();
    }
    if (mode == 1) {
        k_pattern_values<kTableNorm><<<a.groups, threads, 0, st>>>(W, nullptr, s.table, rmean, rvar, gamma, beta, bias, O, lut_binarize);
        BB200_CUDA(cudaPeekAtLastError());
        a.table = s.table;
        k_f32_binary_forward<kPassDirect><<<(unsigned)blocks, threads, 0, st>>>(a);
        return launch_status();
    }
    k_pattern_values<kTableNone><<<a.groups, threads, 0, st>>>(W, s.Y, nullptr, nullptr, nullptr, 0.0f, 0.0f, bias, O, lut_binarize);
    BB200_CUDA(cudaPeekAtLastError());
    BB200_CUDA(cudaMemsetAsync(s.hist, 0, (size_t)O * 256, st));
    a.pat = s.pat;
    k_f32_binary_forward<kPassCount><<<(unsigned)blocks, threads, 0, st>>>(a);
    BB200_CUDA(cudaPeekAtLastError());
    k_dl6_bit_train_finalize<<<a.groups, threads, 0, st>>>(s.Y, s.hist, s.table, mean, rstd, rmean, rvar, gamma, beta, momentum, O, F);
    BB200_CUDA(cudaPeekAtLastError());
    a.table = s.table;
    k_f32_binary_forward<kPassOutput><<<(unsigned)blocks, threads, 0, st>>>(a);
    return launch_status();
}

// Backward of the bit-input layers (StochasticLut6: bn = false; DifferentiableLut6: bn = true).  dx must be zero on entry.
int bit_backward_by_table(bool bn, bool x_is_fp32, const void *x, const float *dy, float *dx, const int *idx, const float *W, float *dW,
                          const float *mean, const float *rstd, float *dmean_out, float *dvar_out, float gamma, float beta, float bias, int O, int F,
                          long long xs, long long fs, int lut_binarize, cudaStream_t st)
{
    if (x_is_fp32 && xs != fs) return BBCU_ERR_NO_MEMORY;          // fp32 x shares the stride of dy / dx in every caller; otherwise decline
    if (O == 0 || F == 0) return BBCU_OK;
    const size_t pat_bytes = (x_is_fp32 && bn) ? (size_t)O * (size_t)fs : 0;      // pattern bytes handed from the histogram pass to the dx pass
    if (pat_bytes > ((size_t)1 << 30)) return BBCU_ERR_NO_MEMORY;
    Scratch s;
    if (!carve(s, O, st, pat_bytes)) return BBCU_ERR_NO_MEMORY;
    float *hdy = reinterpret_cast<float *>(s.hist) + (size_t)O * 64;       // the block between the pattern counts and the truth tables
    BitBwdArgs a = {};
    a.x = static_cast<const uint32_t *>(x); a.dy = dy; a.dx = dx; a.idx = idx; a.W = W; a.hdy = hdy; a.hist = s.hist; a.pat = pat_bytes ? s.pat : nullptr;
    a.mean = mean; a.rstd = rstd; a.dmean = dmean_out; a.dvar = dvar_out;
    a.gamma = gamma; a.beta = beta; a.bias = bias; a.rF = 1.0f / (float)F;
    a.O = O; a.F = F; a.xs = xs; a.fs = fs; a.lut_binarize = lut_binarize;
    a.groups = (O + kWarpsPerCta - 1) / kWarpsPerCta;
    const int words = (F + 31) / 32;
    // tiles of 4096 frames unless that leaves the GPU short of CTAs (each warp pays ~1000 instructions of table set-up per tile)
    a.tile_words = 128;
    while (a.tile_words > 32 && (long long)a.groups * ((words + a.tile_words - 1) / a.tile_words) < 2LL * device_info().sm_count) a.tile_words /= 2;
    const long long blocks = (long long)a.groups * ((words + a.tile_words - 1) / a.tile_words);
    BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
    BB200_CUDA(cudaMemsetAsync(hdy, 0, (size_t)O * 256, st));
    const unsigned nb = (unsigned)blocks, threads = kWarpsPerCta * 32;
    if (!bn) {
        if (x_is_fp32) k_bit_backward_frames<kBwdPlainAll, true><<<nb, threads, 0, st>>>(a);
        else           k_bit_backward_frames<kBwdPlainAll, false><<<nb, threads, 0, st>>>(a);
        BB200_CUDA(cudaPeekAtLastError());
        k_bit_backward_finalize<false><<<a.groups, threads, 0, st>>>(hdy, nullptr, nullptr, dW, nullptr, nullptr, nullptr, nullptr, 0.0f, 0.0f, bias, O, 0.0f, nullptr, nullptr);
        return launch_status();
    }
    k_pattern_values<kTableNone><<<a.groups, threads, 0, st>>>(W, s.Y, nullptr, nullptr, nullptr, 0.0f, 0.0f, bias, O, lut_binarize);
    BB200_CUDA(cudaPeekAtLastError());
    BB200_CUDA(cudaMemsetAsync(s.hist, 0, (size_t)O * 256, st));
    if (!x_is_fp32) {                                   // fp32 frames: the histogram pass below counts the patterns itself
        int tw = 4096;
        while (tw > 32 && (long long)a.groups * ((words + tw - 1) / tw) < 2LL * device_info().sm_count) tw /= 2;
        const long long hb = (long long)a.groups * ((words + tw - 1) / tw);
        k_pattern_histogram<<<(unsigned)hb, threads, 0, st>>>(a.x, idx, s.hist, O, F, xs, a.groups, tw);
        BB200_CUDA(cudaPeekAtLastError());
    }
    if (x_is_fp32) k_bit_backward_frames<kBwdHistOnly, true><<<nb, threads, 0, st>>>(a);
    else           k_bit_backward_frames<kBwdHistOnly, false><<<nb, threads, 0, st>>>(a);
    BB200_CUDA(cudaPeekAtLastError());
    k_bit_backward_finalize<true><<<a.groups, threads, 0, st>>>(hdy, s.hist, s.Y, dW, mean, rstd, dmean_out, dvar_out, gamma, beta, bias, O, 1.0f / (float)F, nullptr, nullptr);
    BB200_CUDA(cudaPeekAtLastError());
    if (x_is_fp32) k_bit_backward_frames<kBwdNormDx, true><<<nb, threads, 0, st>>>(a);
    else           k_bit_backward_frames<kBwdNormDx, false><<<nb, threads, 0, st>>>(a);
    return launch_status();
}


// ---- the two halves of the batch-norm backward for frame-sharded callers (binary mode; bit rows or fp32 rows)
namespace {

// pass 1: pattern values, pattern counts and per-pattern dy sums (and, for fp32 rows, the pattern bytes) of this rank's frames
int backward_pass_one(bool x_is_fp32, BitBwdArgs &a, Scratch &s, float *&hdy, const void *x, const float *dy, const int *idx, const float *W,
                      float bias, int O, int F, long long xs, long long fs, int lut_binarize, cudaStream_t st, bool reuse)
{
    const size_t pat_bytes = x_is_fp32 ? (size_t)O * (size_t)fs : 0;
    if (pat_bytes > ((size_t)1 << 30)) return BBCU_ERR_NO_MEMORY;
    bool have = false;
    if (reuse) {
        std::lock_guard<std::mutex> g(g_record_mu);
        auto it = g_records.find(record_key(st));
        have = it != g_records.end() && it->second.x == x && it->second.dy == dy && it->second.W == W && it->second.O == O && it->second.F == F &&
               it->second.fs == fs;
    }
    if (!carve(s, O, st, pat_bytes)) return BBCU_ERR_NO_MEMORY;           // same size as before: the same block (and it forgets the record)
    hdy = reinterpret_cast<float *>(s.hist) + (size_t)O * 64;
    a = BitBwdArgs{};
    a.x = static_cast<const uint32_t *>(x); a.dy = dy; a.idx = idx; a.W = W; a.hdy = hdy; a.hist = s.hist; a.pat = pat_bytes ? s.pat : nullptr;
    a.bias = bias; a.O = O; a.F = F; a.xs = xs; a.fs = fs; a.lut_binarize = lut_binarize;
    a.groups = (O + kWarpsPerCta - 1) / kWarpsPerCta;
    const int words = (F + 31) / 32;
    a.tile_words = 128;
    while (a.tile_words > 32 && (long long)a.groups * ((words + a.tile_words - 1) / a.tile_words) < 2LL * device_info().sm_count) a.tile_words /= 2;
    const long long blocks = (long long)a.groups * ((words + a.tile_words - 1) / a.tile_words);
    BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
    if (!have) {
        const unsigned threads = kWarpsPerCta * 32;
        BB200_CUDA(cudaMemsetAsync(hdy, 0, (size_t)O * 256, st));
        k_pattern_values<kTableNone><<<a.groups, threads, 0, st>>>(W, s.Y, nullptr, nullptr, nullptr, 0.0f, 0.0f, bias, O, lut_binarize);
        BB200_CUDA(cudaPeekAtLastError());
        BB200_CUDA(cudaMemsetAsync(s.hist, 0, (size_t)O * 256, st));
        if (!x_is_fp32) {
            int tw = 4096;
            while (tw > 32 && (long long)a.groups * ((words + tw - 1) / tw) < 2LL * device_info().sm_count) tw /= 2;
            const long long hb = (long long)a.groups * ((words + tw - 1) / tw);
            k_pattern_histogram<<<(unsigned)hb, threads, 0, st>>>(a.x, idx, s.hist, O, F, xs, a.groups, tw);
            BB200_CUDA(cudaPeekAtLastError());
        }
        if (x_is_fp32) k_bit_backward_frames<kBwdHistOnly, true><<<(unsigned)blocks, threads, 0, st>>>(a);
        else           k_bit_backward_frames<kBwdHistOnly, false><<<(unsigned)blocks, threads, 0, st>>>(a);
        BB200_CUDA(cudaPeekAtLastError());
    }
    return BBCU_OK;
}

}   // namespace

// Statistics half: this rank's (dstd, dmeanx) per node into `sums` ([O][2] fp64), to be added over the ranks by the caller.
int bit_backward_stats_by_table(bool x_is_fp32, const void *x, const float *dy, const int *idx, const float *W, const float *mean, const float *rstd,
                                double *sums, float gamma, float beta, float bias, int O, int F, long long xs, long long fs, int lut_binarize,
                                cudaStream_t st)
{
    if (x_is_fp32 && xs != fs) return BBCU_ERR_NO_MEMORY;
    if (O == 0) return BBCU_OK;
    if (F == 0) { BB200_CUDA(cudaMemsetAsync(sums, 0, sizeof(double) * 2 * (size_t)O, st)); return BBCU_OK; }
    BitBwdArgs a;
    Scratch s;
    float *hdy = nullptr;
    int rc = backward_pass_one(x_is_fp32, a, s, hdy, x, dy, idx, W, bias, O, F, xs, fs, lut_binarize, st, false);
    if (rc) return rc;
    k_bit_backward_finalize<true><<<a.groups, kWarpsPerCta * 32, 0, st>>>(hdy, s.hist, s.Y, nullptr, mean, rstd, nullptr, nullptr, gamma, beta, bias, O,
                                                                          0.0f, sums, nullptr);
    rc = launch_status();
    if (rc == BBCU_OK) {
        PassOneRecord r;
        r.x = x; r.dy = dy; r.W = W; r.O = O; r.F = F; r.fs = fs;
        std::lock_guard<std::mutex> g(g_record_mu);
        g_records[record_key(st)] = r;
    }
    return rc;
}

// Apply half: `sums` hold (dstd, dmeanx) over the frames of ALL ranks, total_frames is their number.  dx must be zero on entry;
// dW receives this rank's share.
int bit_backward_apply_by_table(bool x_is_fp32, const void *x, const float *dy, float *dx, const int *idx, const float *W, float *dW, const float *mean,
                                const float *rstd, const double *sums, float *dmean_out, float *dvar_out, float gamma, float beta, float bias, int O,
                                int F, long long xs, long long fs, long long total_frames, int lut_binarize, cudaStream_t st)
{
    if (x_is_fp32 && xs != fs) return BBCU_ERR_NO_MEMORY;
    if (O == 0 || F == 0) return BBCU_OK;
    BitBwdArgs a;
    Scratch s;
    float *hdy = nullptr;
    int rc = backward_pass_one(x_is_fp32, a, s, hdy, x, dy, idx, W, bias, O, F, xs, fs, lut_binarize, st, true);
    if (rc) return rc;
    const float rF = 1.0f / (float)total_frames;
    const unsigned threads = kWarpsPerCta * 32;
    k_bit_backward_finalize<true><<<a.groups, threads, 0, st>>>(hdy, s.hist, s.Y, dW, mean, rstd, dmean_out, dvar_out, gamma, beta, bias, O, rF, nullptr,
                                                                sums);
    BB200_CUDA(cudaPeekAtLastError());
    a.dx = dx; a.mean = mean; a.rstd = rstd; a.dmean = dmean_out; a.dvar = dvar_out; a.gamma = gamma; a.beta = beta; a.rF = rF;
    const long long blocks = (long long)a.groups * (((F + 31) / 32 + a.tile_words - 1) / a.tile_words);
    if (x_is_fp32) k_bit_backward_frames<kBwdNormDx, true><<<(unsigned)blocks, threads, 0, st>>>(a);
    else           k_bit_backward_frames<kBwdNormDx, false><<<(unsigned)blocks, threads, 0, st>>>(a);
    return launch_status();
}

}   // namespace bb200
