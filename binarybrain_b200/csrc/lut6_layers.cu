// StochasticLut6 and DifferentiableLut6 operators (forward, backward, fp32 and bit-packed inputs).
//
// Results follow the reference's CPU branches:
//   StochasticLutN      include/bb/StochasticLutN.h:512-559 (forward), :668-752 (backward)
//   DifferentiableLutN  include/bb/DifferentiableLutN.h:747-905 (forward), :1157-1266 (backward)
// i.e. no gradient zeroing at x in {0,1} and no clamp of the raw LUT value before batch norm, both of
// which the reference's old CUDA kernels do (cuda/StochasticLut.cuh:191-193,430-470) and its CPU code does not.
//
// Schedule: a CTA is 8 warps = 8 consecutive output nodes working on one frame tile; consecutive CTAs
// walk the node groups of the SAME frame tile, so in the forward kernels the input rows of that tile are fetched
// from HBM once or twice and otherwise hit in L2 for the other nodes that read them.
// Bit-input operators go through per-node pattern tables instead (binary_mode.cu); the kernels here are their fallback.
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "async_copy.cuh"
#include "lut6_core.cuh"

namespace bb200 {

enum Phase {
    PH_PLAIN = 0,   // y = clip(raw, 0, 1)           (bit out: raw > 0.5)
    PH_STATS = 1,   // per-node sum(raw), sum(raw^2) into fp64 sums; fp32 out: raw stored for the normalise pass
    PH_NORM  = 2,   // y = act((raw - mean) * rstd * gamma + beta)
    PH_BWD   = 3,   // pipelined kernel only: the two batch-norm sums of the backward pass from a re-evaluated raw value and dy; no output
};

struct FwdArgs {
    const void *x;          // float or uint32 rows
    float      *y;          // fp32 out (may be null in PH_STATS for bit output)
    uint32_t   *ybits;      // bit out
    const int  *idx;
    const float *W;
    const float *mean;      // PH_NORM
    const float *rstd;      // PH_NORM: rstd, or the running variance when stat_is_var
    double     *sums;       // PH_STATS: [O][2]
    float gamma, beta, bias;
    int O, F, T;
    long long xs, ys;       // row strides in elements (floats / words)
    int lut_binarize, binary, stat_is_var, groups;
    const float *dy;        // PH_BWD: the output gradient, rows of dys floats
    long long dys;
    const float4 *coef;     // pipelined kernel only: per-node tables already in packed-operand form, or nullptr
    int no_scratch;         // launcher: do not take the coefficient table from the stream's scratch (which may allocate)
};

// Centred, conditioned inputs u = x - 1/2 of the lane's four frames of one 128-frame iteration.
template <bool XBIT>
__device__ __forceinline__ void gather_x(float (&xv)[4][6], const void *x, long long xs, const int (&rows)[6], int base, int lane, int F,
                                         int binary, float bias)
{
    if (XBIT) {
        const uint32_t *xw = static_cast<const uint32_t *>(x);
#pragma unroll
        for (int j = 0; j < 6; ++j) {
            const uint32_t *row = xw + (size_t)rows[j] * xs + (base >> 5);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t w = (base + 32 * q < F) ? __ldg(row + q) : 0u;
                xv[q][j] = ((w >> lane) & 1u) ? bias : -bias;
            }
        }
    } else {
        const float *xf = static_cast<const float *>(x);
#pragma unroll
        for (int j = 0; j < 6; ++j) {
            const float *row = xf + (size_t)rows[j] * xs + base + lane;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float v = (base + 32 * q + lane < F) ? __ldg(row + 32 * q) : 0.0f;
                xv[q][j] = condition_u(v, binary, bias);
            }
        }
    }
}

// The same gather split in two: the raw loads (fp32 bit patterns or 32-frame words) and, later, their conditioning.  Keeping the two
// apart lets a kernel issue the loads of its next iteration early and touch the values only when it needs them.
template <bool XBIT>
__device__ __forceinline__ void gather_raw(uint32_t (&raw)[4][6], const void *x, long long xs, const int (&rows)[6], int base, int lane, int F)
{
#pragma unroll
    for (int j = 0; j < 6; ++j) {
        if (XBIT) {
            const uint32_t *row = static_cast<const uint32_t *>(x) + (size_t)rows[j] * xs + (base >> 5);
#pragma unroll
            for (int q = 0; q < 4; ++q) raw[q][j] = (base + 32 * q < F) ? __ldg(row + q) : 0u;
        } else {
            const uint32_t *row = static_cast<const uint32_t *>(x) + (size_t)rows[j] * xs + base + lane;
#pragma unroll
            for (int q = 0; q < 4; ++q) raw[q][j] = (base + 32 * q + lane < F) ? __ldg(row + 32 * q) : 0u;
        }
    }
}

// fp32 rows addressed by ready-made element offsets (row * stride), so that the per-access address is one 64-bit add
__device__ __forceinline__ void gather_raw_off(uint32_t (&raw)[4][6], const float *x, const long long (&off)[6], int base, int lane, int F)
{
#pragma unroll
    for (int j = 0; j < 6; ++j) {
        const uint32_t *row = reinterpret_cast<const uint32_t *>(x + off[j]) + base + lane;
#pragma unroll
        for (int q = 0; q < 4; ++q) raw[q][j] = (base + 32 * q + lane < F) ? __ldg(row + 32 * q) : 0u;
    }
}

template <bool XBIT>
__device__ __forceinline__ void condition_raw(float (&xv)[4][6], const uint32_t (&raw)[4][6], int lane, int binary, float bias)
{
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int j = 0; j < 6; ++j)
            xv[q][j] = XBIT ? (((raw[q][j] >> lane) & 1u) ? bias : -bias) : condition_u(__uint_as_float(raw[q][j]), binary, bias);
}

constexpr int kFwdCtas = 2;   // resident CTAs per SM the forward kernels are compiled for (register cap 65536 / (256 * n))

template <bool XBIT, int PHASE, bool YBIT>
__global__ void __launch_bounds__(kWarpsPerCta * 32, kFwdCtas)
k_lut6_forward(const FwdArgs a)
{
    __shared__ float4 s_tab[kWarpsPerCta][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / a.groups;
    const int node = (blockIdx.x % a.groups) * kWarpsPerCta + warp;
    if (node >= a.O) return;

    float4 *tab = s_tab[warp];
    stage_table_x2(tab, a.W, node, lane, a.lut_binarize);
    int rows[6];
#pragma unroll
    for (int j = 0; j < 6; ++j) rows[j] = __ldg(a.idx + (size_t)node * 6 + j);

    float mean = 0.0f, scale = 0.0f;
    if (PHASE == PH_NORM) {
        mean = a.mean[node];
        float r = a.rstd[node];
        if (a.stat_is_var) r = 1.0f / sqrtf(r);        // DifferentiableLutN.h:866-868
        scale = r;
    }
    double s1 = 0.0, s2 = 0.0;

    const int f_begin = tile * a.T;
    const int f_end   = min(a.F, f_begin + a.T);
    for (int base = f_begin; base < f_end; base += kFramesPerIter) {
        float xv[4][6];
        gather_x<XBIT>(xv, a.x, a.xs, rows, base, lane, a.F, a.binary, a.bias);
        // frames q = 0,1 and q = 2,3 of this lane travel as two packed pairs through one walk of the tree
        f32x2 xp[6][2], yp[2];
#pragma unroll
        for (int j = 0; j < 6; ++j) { xp[j][0] = pack2(xv[0][j], xv[1][j]); xp[j][1] = pack2(xv[2][j], xv[3][j]); }
        lut6_forward_x2<2>(tab, xp, yp);
        float vq[4];
        unpack2(yp[0], vq[0], vq[1]);
        unpack2(yp[1], vq[2], vq[3]);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int f = base + 32 * q + lane;
            const bool live = f < a.F;
            float v = vq[q];
            if (PHASE == PH_STATS) {
                if (live) { s1 += (double)v; s2 += (double)v * (double)v; }
                if (!YBIT && live) a.y[(size_t)node * a.ys + f] = v;
            } else {
                if (PHASE == PH_NORM) {
                    v = (v - mean) * scale;
                    v = v * a.gamma + a.beta;
                }
                if (YBIT) {
                    unsigned m = __ballot_sync(kFull, live && v > 0.5f);
                    if (lane == 0 && base + 32 * q < a.F) a.ybits[(size_t)node * a.ys + ((base >> 5) + q)] = m;
                } else if (live) {
                    if (PHASE == PH_NORM && a.binary) v = v > 0.5f ? 1.0f : 0.0f;
                    else                              v = __saturatef(v);
                    a.y[(size_t)node * a.ys + f] = v;
                }
            }
        }
    }
    if (PHASE == PH_STATS) {
        s1 = warp_sum(s1);
        s2 = warp_sum(s2);
        if (lane == 0) {
            atomicAdd(a.sums + 2 * (size_t)node, s1);
            atomicAdd(a.sums + 2 * (size_t)node + 1, s2);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Persistent, copy-pipelined forward for fp32 inputs with 16-byte aligned rows (the launcher's default).
// Work item = (frame tile of a.T = 128 or 256 frames, group of 8 nodes); CTA c takes items c, c + gridDim, ... so
// the CTAs in flight sweep the node groups of one tile together and the tile's rows stay in L2.  Each warp owns one
// node of the group and runs its own two-stage pipeline of cp.async copies: every lane copies the 16-byte pieces of the six
// gathered row segments that it will itself read (frames 128 h + 4 lane .. + 3) and one piece of the node's table, for item
// j+2 once item j has been read out of shared memory, and the warp computes item j while the copies of j+1 (and j+2) are in
// flight.  (Bulk copies with an mbarrier did the same with seven copy instructions per item, but each of them cost five moves
// into uniform registers plus the election of the issuing lane: a fifth of the kernel's issue slots.)
// The table normally arrives ready to use: a small kernel in front (k_table_coeffs) has turned every node's 64 entries
// into the 32 x (c0, c0, c1, c1) packed-operand form once per launch, so no warp repeats that butterfly (ten shuffles
// in a dependent chain) for every item.  Tables have a ring of three slots per warp because the table of item j is
// still being read while the copies of item j+2 are started.  Without the scratch table (a.coef == nullptr) the raw
// entries are copied instead and converted in place.
// ---------------------------------------------------------------------------------------------
constexpr int kFpMaxItemFrames = 256;          // 128-frame items with three CTAs per SM (80 registers) measured 20 % slower
constexpr int kFpCtas          = 2;
constexpr int kFpStages        = 2;
constexpr int kFpStageBytes    = 6 * kFpMaxItemFrames * 4;                             // six row segments
constexpr int kFpRowsBytes     = kWarpsPerCta * kFpStages * kFpStageBytes;
constexpr int kFpTabSlots      = 3;
constexpr int kFpTabSlotBytes  = 32 * 16;
constexpr int kFpTabBytes      = kWarpsPerCta * kFpTabSlots * kFpTabSlotBytes;
constexpr int kFpSmem          = kFpRowsBytes + kFpTabBytes;
static_assert(kFpCtas * (kFpSmem + 1024) <= 227 * 1024, "the CTAs of one SM must fit");

// Position of a work item, advanced incrementally (item index + gridDim) so that no division runs per item.
struct FpPos {
    int tile, group;
};

__device__ __forceinline__ FpPos fp_advance(FpPos p, int dt, int dg, int groups)
{
    p.group += dg;
    p.tile += dt;
    if (p.group >= groups) { p.group -= groups; ++p.tile; }
    return p;
}

// The copies of input rows J..5 of an item: one shuffle and one 64-bit multiply-add per row, offsets as immediates.
template <int J, bool TWO>
struct FpRowCopies {
    static __device__ __forceinline__ void issue(uint32_t sb, uint64_t gb, int row, size_t row_bytes)
    {
        const uint64_t src = gb + (uint64_t)__shfl_sync(0xffffffffu, row, J) * row_bytes;
        cp_async16_at<J * kFpMaxItemFrames * 4, 0>(sb, src);
        if (TWO) cp_async16_at<J * kFpMaxItemFrames * 4 + kFramesPerIter * 4, kFramesPerIter * 4>(sb, src);
        FpRowCopies<J + 1, TWO>::issue(sb, gb, row, row_bytes);
    }
};
template <bool TWO>
struct FpRowCopies<6, TWO> {
    static __device__ __forceinline__ void issue(uint32_t, uint64_t, int, size_t) {}
};

// `row` is the lane's input row of the item's node (lanes 0..5; fp_row), fetched an item earlier so that the copies do not wait
// for it.  One commit group per call, whether or not the item exists, so that the consumer's wait counts items.
__device__ __forceinline__ int fp_row(const FwdArgs &a, FpPos pos, int warp, int lane)
{
    const int node = min(pos.group * kWarpsPerCta + warp, a.O - 1);
    return lane < 6 ? __ldg(a.idx + (size_t)node * 6 + lane) : 0;
}

__device__ __forceinline__ void fp_issue(const FwdArgs &a, FpPos pos, bool exists, int row, int warp, int lane, unsigned char *stage,
                                         unsigned char *tab_slot)
{
    if (exists) {
        const int node = min(pos.group * kWarpsPerCta + warp, a.O - 1);
        const int f0 = pos.tile * a.T;
        const size_t row_bytes = (size_t)a.xs * 4;
        const unsigned char *xb = static_cast<const unsigned char *>(a.x) + ((size_t)f0 + 4 * lane) * 4;      // this lane's first piece of row 0
        unsigned char *dst = stage + 16 * lane;
        constexpr int kRow = kFpMaxItemFrames * 4, kHalf = kFramesPerIter * 4;
        if (f0 + a.T <= a.xs) {                                                 // every piece of the item lies inside the rows (all but a last tile)
            const uint32_t sb = smem_addr(dst);
            const uint64_t gb = (uint64_t)__cvta_generic_to_global(xb);
            if (a.T > kFramesPerIter) FpRowCopies<0, true>::issue(sb, gb, row, row_bytes);
            else                      FpRowCopies<0, false>::issue(sb, gb, row, row_bytes);
        } else {
#pragma unroll
            for (int j = 0; j < 6; ++j) {
                const unsigned char *src = xb + (size_t)__shfl_sync(kFull, row, j) * row_bytes;
#pragma unroll
                for (int h = 0; h < kFpMaxItemFrames / kFramesPerIter; ++h) {
                    if (kFramesPerIter * h < a.T) {                             // (a.T is 128 or 256)
                        const bool in_row = f0 + 4 * lane + kFramesPerIter * h < a.xs;      // row stride is a multiple of 4 floats
                        cp_async16(dst + j * kRow + h * kHalf, in_row ? src + h * kHalf : static_cast<const unsigned char *>(a.x), in_row);
                    }
                }
            }
        }
        if (a.coef)         cp_async16(tab_slot + 16 * lane, a.coef + (size_t)node * 32 + lane, true);
        else if (lane < 16) cp_async16(tab_slot + 16 * lane, a.W + (size_t)node * 64 + 4 * lane, true);
    }
    cp_async_commit();
}

// Every node's table as 32 x (c0, c0, c1, c1): the polynomial coefficients, each duplicated for the two halves of a packed operand.
__global__ void __launch_bounds__(kWarpsPerCta * 32)
k_table_coeffs(const float *__restrict__ W, float4 *__restrict__ coef, int O, int lut_binarize)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int node = blockIdx.x * kWarpsPerCta + warp;
    if (node >= O) return;
    float2 v = reinterpret_cast<const float2 *>(W + (size_t)node * 64)[lane];
    if (lut_binarize) { v.x = v.x > 0.5f ? 1.0f : 0.0f; v.y = v.y > 0.5f ? 1.0f : 0.0f; }
    v = table_to_coeffs(v, lane);
    coef[(size_t)node * 32 + lane] = make_float4(v.x, v.x, v.y, v.y);
}

template <int PHASE, bool BINARY>            // BINARY: the layer's binary mode, compiled in so that input conditioning is one instruction
__global__ void __launch_bounds__(kWarpsPerCta * 32, kFpCtas)
k_lut6_forward_pipe(const FwdArgs a, int n_tiles)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char *my_stages = smem_raw + (size_t)warp * kFpStages * kFpStageBytes;
    unsigned char *my_tabs = smem_raw + kFpRowsBytes + (size_t)warp * kFpTabSlots * kFpTabSlotBytes;

    // items blockIdx, blockIdx + gridDim, ...: position of the current item and of the next two
    const int step = (int)gridDim.x;
    const int dt = step / a.groups, dg = step - dt * a.groups;
    FpPos p0;
    p0.tile  = (int)blockIdx.x / a.groups;
    p0.group = (int)blockIdx.x - p0.tile * a.groups;
    FpPos p1 = fp_advance(p0, dt, dg, a.groups);
    FpPos p2 = fp_advance(p1, dt, dg, a.groups);
    fp_issue(a, p0, p0.tile < n_tiles, p0.tile < n_tiles ? fp_row(a, p0, warp, lane) : 0, warp, lane, my_stages, my_tabs);
    fp_issue(a, p1, p1.tile < n_tiles, p1.tile < n_tiles ? fp_row(a, p1, warp, lane) : 0, warp, lane, my_stages + kFpStageBytes,
             my_tabs + kFpTabSlotBytes);
    int row2 = p2.tile < n_tiles ? fp_row(a, p2, warp, lane) : 0;            // input rows of item k+2, one item ahead of their use
    int ts = 0;                                   // table slot of the current item: k mod 3

    // per-node batch-norm constants travel one item ahead of their use
    float mean_n = 0.0f, scale_n = 0.0f;
    if ((PHASE == PH_NORM || PHASE == PH_BWD) && p0.tile < n_tiles) {
        const int n0 = min(p0.group * kWarpsPerCta + warp, a.O - 1);
        mean_n = a.mean[n0];
        scale_n = a.rstd[n0];
    }

    for (int k = 0; p0.tile < n_tiles; ++k) {
        const int s = k & 1;
        unsigned char *stage = my_stages + s * kFpStageBytes;
        const int node_raw = p0.group * kWarpsPerCta + warp;
        const bool store = node_raw < a.O;
        const int node = min(node_raw, a.O - 1);
        const int f0 = p0.tile * a.T;
        const int nf = min(a.T, a.F - f0);
        float mean = mean_n, scale = scale_n;
        if (PHASE == PH_NORM && a.stat_is_var) scale = 1.0f / sqrtf(scale);        // DifferentiableLutN.h:866-868
        const bool have_next = p1.tile < n_tiles;
        if ((PHASE == PH_NORM || PHASE == PH_BWD) && have_next) {
            const int n1 = min(p1.group * kWarpsPerCta + warp, a.O - 1);
            mean_n = a.mean[n1];
            scale_n = a.rstd[n1];
        }

        cp_async_wait<1>();                            // this item's group has landed (the next item's may still be in flight)
        __syncwarp();                                  // the table was copied by other lanes
        float4 *tab = reinterpret_cast<float4 *>(my_tabs + ts * kFpTabSlotBytes);
        unsigned char *tab_refill = my_tabs + (ts == 0 ? 2 : ts - 1) * kFpTabSlotBytes;      // slot (k + 2) mod 3, last read by item k - 1
        ts = ts == 2 ? 0 : ts + 1;
        if (a.coef == nullptr) {   // raw W[64] arrived: convert in place to 32 x (c0, c0, c1, c1)
            float2 v = reinterpret_cast<const float2 *>(tab)[lane];
            if (a.lut_binarize) { v.x = v.x > 0.5f ? 1.0f : 0.0f; v.y = v.y > 0.5f ? 1.0f : 0.0f; }
            v = table_to_coeffs(v, lane);
            __syncwarp();
            tab[lane] = make_float4(v.x, v.x, v.y, v.y);
            __syncwarp();
        }
        double s1 = 0.0, s2 = 0.0;
        const float *xs0 = reinterpret_cast<const float *>(stage);
        float *yrow = PHASE == PH_BWD ? nullptr : a.y + (size_t)node * a.ys + f0 + 4 * lane;
        const float *dyrow = PHASE == PH_BWD ? a.dy + (size_t)node * a.dys + f0 + 4 * lane : nullptr;
        const float rstd2 = scale * scale;                 // PH_BWD
        // One walk of the tree carries NP frame pairs per lane.  A lane owns four consecutive frames of every 128 (frames 128h + 4 lane
        // + 0..3, h < NP/2; pairs (0, 1) and (2, 3)), so its inputs come out of shared memory with one 128-bit load per row and half and
        // its outputs leave with one 128-bit store per half: 4 pairs when the item is 256 frames wide, 2 pairs for a 128-frame item.
        const FpPos p3 = fp_advance(p2, dt, dg, a.groups);
        auto walk = [&](auto np_tag) {
            constexpr int NP = decltype(np_tag)::value;
            f32x2 up[6][NP], yp[NP];
            float g4[NP / 2][4];                                   // PH_BWD: dy of the lane's frames, fetched ahead of the tree
            if (PHASE == PH_BWD) {
#pragma unroll
                for (int h = 0; h < NP / 2; ++h) {
                    const int fl = 128 * h + 4 * lane;
                    if (fl + 3 < nf) {
                        const float4 q = __ldg(reinterpret_cast<const float4 *>(dyrow + 128 * h));
                        g4[h][0] = q.x; g4[h][1] = q.y; g4[h][2] = q.z; g4[h][3] = q.w;
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) g4[h][i] = fl + i < nf ? __ldg(dyrow + 128 * h + i) : 0.0f;
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 6; ++j) {
#pragma unroll
                for (int h = 0; h < NP / 2; ++h) {
                    const float4 r = *reinterpret_cast<const float4 *>(xs0 + j * kFpMaxItemFrames + 128 * h + 4 * lane);
                    // the same values as condition_u()
                    if (BINARY) {
                        up[j][2 * h]     = pack2(r.x > 0.5f ? a.bias : -a.bias, r.y > 0.5f ? a.bias : -a.bias);
                        up[j][2 * h + 1] = pack2(r.z > 0.5f ? a.bias : -a.bias, r.w > 0.5f ? a.bias : -a.bias);
                    } else {
                        up[j][2 * h]     = pack2(__saturatef(r.x) - 0.5f, __saturatef(r.y) - 0.5f);
                        up[j][2 * h + 1] = pack2(__saturatef(r.z) - 0.5f, __saturatef(r.w) - 0.5f);
                    }
                }
            }
            // the stage has been read out: hand it back to the copy engine for item k+2 before doing the math
            __syncwarp();
            fp_issue(a, p2, p2.tile < n_tiles, row2, warp, lane, stage, tab_refill);
            if (p3.tile < n_tiles) row2 = fp_row(a, p3, warp, lane);
            lut6_forward_x2<NP>(tab, up, yp);
#pragma unroll
            for (int h = 0; h < NP / 2; ++h) {
                float v[4];
                unpack2(yp[2 * h], v[0], v[1]);
                unpack2(yp[2 * h + 1], v[2], v[3]);
                const int fl = 128 * h + 4 * lane;                 // first of the lane's four frames, relative to the item
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (PHASE == PH_STATS) {
                        if (store && fl + i < nf) { s1 += (double)v[i]; s2 += (double)v[i] * (double)v[i]; }
                    } else if (PHASE == PH_BWD) {
                        if (store && fl + i < nf) {                // DifferentiableLutN.h:1190-1215, as k_lut6_backward_stats
                            const float tanh_x = ((v[i] - mean) * scale) * a.gamma + a.beta;
                            float g = g4[h][i];
                            if (tanh_x <= 0.0f || tanh_x >= 1.0f) g = 0.0f;
                            const float dxn = a.gamma * g;
                            s1 -= (double)(dxn * (v[i] - mean) * rstd2);
                            s2 -= (double)(dxn * scale);
                        }
                    } else if (PHASE == PH_NORM) {
                        v[i] = (v[i] - mean) * scale;
                        v[i] = v[i] * a.gamma + a.beta;
                        v[i] = BINARY ? (v[i] > 0.5f ? 1.0f : 0.0f) : __saturatef(v[i]);
                    } else {
                        v[i] = __saturatef(v[i]);
                    }
                }
                if (store && PHASE != PH_BWD) {
                    if (fl + 3 < nf) {
                        *reinterpret_cast<float4 *>(yrow + 128 * h) = make_float4(v[0], v[1], v[2], v[3]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 3; ++i)
                            if (fl + i < nf) yrow[128 * h + i] = v[i];
                    }
                }
            }
        };
        if (kFpMaxItemFrames > kFramesPerIter && nf > kFramesPerIter) walk(std::integral_constant<int, kFpMaxItemFrames / 64>());
        else                                                          walk(std::integral_constant<int, 2>());
        if ((PHASE == PH_STATS || PHASE == PH_BWD) && store) {
            s1 = warp_sum(s1);
            s2 = warp_sum(s2);
            if (lane == 0) {
                atomicAdd(a.sums + 2 * (size_t)node, s1);
                atomicAdd(a.sums + 2 * (size_t)node + 1, s2);
            }
        }
        p0 = p1; p1 = p2; p2 = p3;
    }
    cp_async_wait<0>();
}

// mean / var / rstd and the running statistics from the fp64 sums (DifferentiableLutN.h:804-812).
__global__ void k_bn_finalize(const double *__restrict__ sums, float *mean_out, float *rstd_out, float *running_mean, float *running_var,
                              float momentum, int O, long long total_frames)
{
    int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= O) return;
    const float rF   = 1.0f / (float)total_frames;
    const float s1   = (float)sums[2 * (size_t)n];
    const float s2   = (float)sums[2 * (size_t)n + 1];
    const float mean = s1 * rF;
    // one fused multiply-subtract, which is what the reference's build flags make of (s2*rF) - (mean*mean)
    const float var  = fmaxf(1.0e-5f, fmaf(s2, rF, -(mean * mean)));
    const float rstd = 1.0f / sqrtf(var);
    running_mean[n] = running_mean[n] * momentum + mean * (1.0f - momentum);
    running_var[n]  = running_var[n]  * momentum + var  * (1.0f - momentum);
    mean_out[n] = mean;
    rstd_out[n] = rstd;
}

// In-place normalise of the raw LUT values stored by PH_STATS: one CTA per (node, 4096-frame chunk).
__global__ void __launch_bounds__(256)
k_bn_normalize_inplace(float *y, const float *__restrict__ mean_buf, const float *__restrict__ rstd_buf, float gamma, float beta,
                       int F, long long ys, int binary, int chunks)
{
    const int node = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    const float mean = mean_buf[node], rstd = rstd_buf[node];
    float *row = y + (size_t)node * ys;
    const int f0 = chunk * 4096;
    const int f1 = min(F, f0 + 4096);
    const bool vec = ((reinterpret_cast<uintptr_t>(row) & 15) == 0);
    if (vec) {
        // all four 128-bit loads of a thread are in flight before the first store (16 KiB per CTA)
        float4 v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int f = f0 + threadIdx.x * 4 + 1024 * k;
            if (f + 3 < f1) v[k] = *reinterpret_cast<const float4 *>(row + f);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int f = f0 + threadIdx.x * 4 + 1024 * k;
            if (f + 3 < f1) {
                float o[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float t = (o[i] - mean) * rstd;
                    t = t * gamma + beta;
                    o[i] = binary ? (t > 0.5f ? 1.0f : 0.0f) : fmaxf(0.0f, fminf(1.0f, t));
                }
                *reinterpret_cast<float4 *>(row + f) = make_float4(o[0], o[1], o[2], o[3]);
            } else {
                for (int g = f; g < f1; ++g) {
                    float t = (row[g] - mean) * rstd;
                    t = t * gamma + beta;
                    row[g] = binary ? (t > 0.5f ? 1.0f : 0.0f) : fmaxf(0.0f, fminf(1.0f, t));
                }
            }
        }
    } else {
        for (int f = f0 + threadIdx.x; f < f1; f += 256) {
            float t = (row[f] - mean) * rstd;
            t = t * gamma + beta;
            row[f] = binary ? (t > 0.5f ? 1.0f : 0.0f) : fmaxf(0.0f, fminf(1.0f, t));
        }
    }
}

// ---------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------
struct BwdArgs {
    const void *x;
    const float *dy;
    float *dx;
    const int *idx;
    const float *W;
    float *dW;
    const float *mean, *rstd;     // batch norm only
    const float *dmean, *dvar;    // batch norm apply pass
    double *sums;                 // batch norm stats pass: [O][2] = (dstd, dmeanx)
    float gamma, beta, bias, rF;
    int O, F, T;
    long long xs, dys, dxs;
    int lut_binarize, binary, groups;
};

// Batch-norm statistics of the backward pass (DifferentiableLutN.h:1190-1220): the hard-tanh mask is
// re-derived from the recomputed forward value; dstd = sum -(g*dy*(raw-mean)*rstd^2), dmeanx = sum -(g*dy*rstd).
template <bool XBIT>
__global__ void __launch_bounds__(kWarpsPerCta * 32, 3)
k_lut6_backward_stats(const BwdArgs a)
{
    __shared__ float4 s_tab[kWarpsPerCta][16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / a.groups;
    const int node = (blockIdx.x % a.groups) * kWarpsPerCta + warp;
    if (node >= a.O) return;
    float4 *tab = s_tab[warp];
    stage_table_halves(tab, a.W, node, lane, a.lut_binarize);
    int rows[6];
#pragma unroll
    for (int j = 0; j < 6; ++j) rows[j] = __ldg(a.idx + (size_t)node * 6 + j);
    const float mean = a.mean[node], rstd = a.rstd[node], rstd2 = rstd * rstd;
    double dstd = 0.0, dmeanx = 0.0;

    const int f_begin = tile * a.T;
    const int f_end   = min(a.F, f_begin + a.T);
    for (int base = f_begin; base < f_end; base += kFramesPerIter) {
        float xv[4][6];
        gather_x<XBIT>(xv, a.x, a.xs, rows, base, lane, a.F, a.binary, a.bias);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int f = base + 32 * q + lane;
            if (f < a.F) {
                float v = lut6_forward_halves(tab, xv[q]);
                float tanh_x = ((v - mean) * rstd) * a.gamma + a.beta;
                float g = __ldg(a.dy + (size_t)node * a.dys + f);
                if (tanh_x <= 0.0f || tanh_x >= 1.0f) g = 0.0f;
                float dxn = a.gamma * g;
                dstd   -= (double)(dxn * (v - mean) * rstd2);
                dmeanx -= (double)(dxn * rstd);
            }
        }
    }
    dstd = warp_sum(dstd);
    dmeanx = warp_sum(dmeanx);
    if (lane == 0) {
        atomicAdd(a.sums + 2 * (size_t)node, dstd);
        atomicAdd(a.sums + 2 * (size_t)node + 1, dmeanx);
    }
}

// Batch-norm statistics of the backward pass from the layer's own OUTPUT instead of a recomputed LUT value (non-binary
// mode only).  y = clip((raw - mean) * rstd * gamma + beta, 0, 1): where y is strictly inside (0, 1) the hard-tanh passes
// the gradient and (raw - mean) * rstd = (y - beta) / gamma, so  -(gamma*dy*(raw - mean)*rstd^2) = -dy*(y - beta)*rstd;
// where y is 0 or 1 the gradient is masked (DifferentiableLutN.h:1204-1206).  An HBM-bound stream over y and dy
// (8 bytes per node-frame) replaces a second evaluation of the LUT tree.
__global__ void __launch_bounds__(256)
k_dl6_backward_stats_from_y(const float *__restrict__ y, const float *__restrict__ dy, const float *__restrict__ rstd_buf, double *sums,
                            float gamma, float beta, int F, long long ys, long long dys, int chunks)
{
    __shared__ double red[2][8];
    const int node = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    const float *yr = y + (size_t)node * ys;
    const float *gr = dy + (size_t)node * dys;
    const int f0 = chunk * 8192, f1 = min(F, f0 + 8192);
    const float rstd = rstd_buf[node];
    double dstd = 0.0, dmeanx = 0.0;
    const bool vec = ((reinterpret_cast<uintptr_t>(yr) | reinterpret_cast<uintptr_t>(gr)) & 15) == 0;
    auto one = [&](float yv, float g) {
        if (yv <= 0.0f || yv >= 1.0f) g = 0.0f;
        dstd   -= (double)(g * (yv - beta) * rstd);
        dmeanx -= (double)((gamma * g) * rstd);
    };
    if (vec) {
        int f = f0 + threadIdx.x * 4;
        for (; f + 3 < f1; f += 1024) {
            const float4 a = __ldg(reinterpret_cast<const float4 *>(yr + f));
            const float4 g = __ldg(reinterpret_cast<const float4 *>(gr + f));
            one(a.x, g.x); one(a.y, g.y); one(a.z, g.z); one(a.w, g.w);
        }
        const int tail = f0 + ((f1 - f0) & ~3);          // the last 0..3 frames of the chunk
        if ((int)threadIdx.x < f1 - tail) one(__ldg(yr + tail + threadIdx.x), __ldg(gr + tail + threadIdx.x));
    } else {
        for (int f = f0 + threadIdx.x; f < f1; f += 256) one(__ldg(yr + f), __ldg(gr + f));
    }
    // block reduction of the two sums
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) { dstd += __shfl_xor_sync(kFull, dstd, m); dmeanx += __shfl_xor_sync(kFull, dmeanx, m); }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { red[0][warp] = dstd; red[1][warp] = dmeanx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        double a = 0.0, b = 0.0;
        for (int w = 0; w < 8; ++w) { a += red[0][w]; b += red[1][w]; }
        atomicAdd(sums + 2 * (size_t)node, a);
        atomicAdd(sums + 2 * (size_t)node + 1, b);
    }
}

__global__ void k_bn_backward_finalize(const double *__restrict__ sums, const float *__restrict__ mean_buf, const float *__restrict__ rstd_buf,
                                       float *dmean_out, float *dvar_out, int O, long long total_frames)
{
    int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= O) return;
    const float rF = 1.0f / (float)total_frames;
    const float dstd = (float)sums[2 * (size_t)n], dmeanx = (float)sums[2 * (size_t)n + 1];
    const float dvar = dstd * rstd_buf[n];
    dvar_out[n]  = dvar;
    dmean_out[n] = (dmeanx - (mean_buf[n] * dvar)) * rF;
}

// dW / dx.  BN = true folds the batch-norm backward (DifferentiableLutN.h:1225-1258) in front of the LUT's.
// dx rows must be zero on entry: every node adds its six input gradients with red.global.add.f32.  With the wide (4096-frame)
// tiles used for the sake of the dW accumulators the tile's dx rows no longer all stay in L2 (ncu: 20 % hit rate), which measured
// cheaper than reducing the 64 accumulators more often.
template <bool XBIT, bool BN>
__global__ void __launch_bounds__(kWarpsPerCta * 32, 1)
k_lut6_backward(const BwdArgs a)
{
    __shared__ float4 s_tab[kWarpsPerCta][16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / a.groups;
    const int node = (blockIdx.x % a.groups) * kWarpsPerCta + warp;
    if (node >= a.O) return;
    float4 *tab = s_tab[warp];
    stage_table_halves(tab, a.W, node, lane, a.lut_binarize);
    // fp32 inputs: x and dx rows share one stride, so one 64-bit element offset per input serves both and an access costs a single
    // 64-bit add; bit inputs keep the row numbers for the (word-strided) x rows as well
    int rows[6];
    long long off[6];
#pragma unroll
    for (int j = 0; j < 6; ++j) {
        rows[j] = __ldg(a.idx + (size_t)node * 6 + j);
        off[j] = (long long)rows[j] * a.dxs;
    }

    float mean = 0.0f, rstd = 0.0f, dmean = 0.0f, dvar_rF = 0.0f;
    if (BN) {
        mean = a.mean[node];
        rstd = a.rstd[node];
        dmean = a.dmean[node];
        dvar_rF = a.dvar[node];
    }
    f32x2 acc2[32];                       // (dC[i], dC[i + 32]): both halves of the tree travel in one packed operand
#pragma unroll
    for (int i = 0; i < 32; ++i) acc2[i] = 0ull;

    const int f_begin = tile * a.T;
    const int f_end   = min(a.F, f_begin + a.T);
    // The loads of iteration i + 1 are issued before the arithmetic of iteration i (about 1000 instructions), so their latency is
    // covered by this warp's own work: with ~240 registers per thread only two warps share a scheduler and cannot cover it for each other.
    uint32_t xn[4][6];
    float dyn[4];
    if (XBIT) gather_raw<true>(xn, a.x, a.xs, rows, f_begin, lane, a.F);
    else      gather_raw_off(xn, static_cast<const float *>(a.x), off, f_begin, lane, a.F);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int f = f_begin + 32 * q + lane;
        dyn[q] = (f < a.F) ? __ldg(a.dy + (size_t)node * a.dys + f) : 0.0f;
    }
    for (int base = f_begin; base < f_end; base += kFramesPerIter) {
        float xv[4][6], dyv[4];
        condition_raw<XBIT>(xv, xn, lane, a.binary, a.bias);
#pragma unroll
        for (int q = 0; q < 4; ++q) dyv[q] = dyn[q];
        if (base + kFramesPerIter < f_end) {
            if (XBIT) gather_raw<true>(xn, a.x, a.xs, rows, base + kFramesPerIter, lane, a.F);
            else      gather_raw_off(xn, static_cast<const float *>(a.x), off, base + kFramesPerIter, lane, a.F);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int f = base + kFramesPerIter + 32 * q + lane;
                dyn[q] = (f < a.F) ? __ldg(a.dy + (size_t)node * a.dys + f) : 0.0f;
            }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int f = base + 32 * q + lane;
            KeptHalves D;
            float v = lut6_forward_keep_halves(tab, xv[q], D);
            float g = dyv[q];
            if (BN) {
                float tanh_x = ((v - mean) * rstd) * a.gamma + a.beta;
                if (tanh_x <= 0.0f || tanh_x >= 1.0f) g = 0.0f;
                float dxc = (g * a.gamma) * rstd;
                g = dxc + dmean + (v * dvar_rF * a.rF);
                if (f >= a.F) g = 0.0f;
            }
            float dxv[6];
            lut6_reverse_halves(tab, xv[q], D, g, acc2, dxv);
            if (f < a.F) {
                float *dxf = a.dx + f;
#pragma unroll
                for (int j = 0; j < 6; ++j) atomicAdd(dxf + off[j], dxv[j]);
            }
        }
    }
    float acc[64];
#pragma unroll
    for (int i = 0; i < 32; ++i) unpack2(acc2[i], acc[i], acc[i + 32]);
    warp_reduce_scatter64(acc, lane);
    const float2 gw = coeff_grads_to_table(make_float2(acc[0], acc[1]), lane);
    float *dst = a.dW + (size_t)node * 64 + 2 * lane;
    atomicAdd(dst, gw.x);
    atomicAdd(dst + 1, gw.y);
}

// ---------------------------------------------------------------------------------------------
// Persistent backward for fp32 frames whose rows start on 16-byte boundaries (the launcher's default).
//
// Work item = (frame tile of a.T frames, group of 8 nodes), walked in tile-major order by one CTA per SM; each warp owns one node
// of the group.  What the kernel is bound by: an SM sub-partition issues one instruction per clock and a packed f32x2
// instruction takes two issue slots (measured: 32 packed FMAs take 65 clocks per warp, and scalar FMAs, logic ops or anything
// else issued beside them add their own clocks in full), so the time is the weighted instruction count -- 113 packed (226
// slots) + about 105 others per frame -- over the issue rate.  Everything here is about the "others":
//   * the per-node table arrives ready to use (k_table_halves has converted every table once per launch);
//   * global -> shared: a warp streams its item in 128-frame chunks through a three-stage ring; every lane copies 16 bytes (four
//     consecutive frames) of each of the six input rows and of dy with cp.async, two chunks ahead of the arithmetic, so the
//     prefetch holds no registers and the loop has no global address arithmetic per frame;
//   * arithmetic: lane l takes the frame pairs 64 h + 2 l + {0, 1}, h = 0, 1, of the chunk: one conflict-free 64-bit shared load
//     per row and pair;
//   * the six input gradients of a pair go to a staging area in shared memory (conflict-free 64-bit stores); after the chunk's
//     four frames every lane adds its four consecutive frames of each row to dx with one 128-bit reduction
//     (red.global.add.v4.f32), which L2 resolves;
//   * at the end of an item the 64 per-lane gradient sums are added across lanes through a padded transpose in shared memory
//     (16 stores, 32 loads and 32 packed adds per lane instead of 62 shuffles with two selects each) and leave as one 8-byte
//     reduction per lane into the coefficient-gradient scratch dC, which k_coeff_grads_to_dw maps to table gradients once per
//     launch.
// The tile is wide (1024-2048 frames) to amortise that flush: measured, the extra L2 misses of a wide tile cost less than
// flushing more often, because the kernel is issue-bound, not memory-bound.
// dx rows must be zero on entry.
// ---------------------------------------------------------------------------------------------
constexpr int kBvStages     = 3;
constexpr int kBvRowBytes   = kFramesPerIter * 4;                 // one row segment of a chunk
constexpr int kBvStageBytes = 7 * kBvRowBytes;                    // six input rows and dy
constexpr int kBvTabSlots   = 3;                                  // the copy side runs at most two items ahead of the arithmetic
constexpr int kBvTabBytes   = 16 * 16;
constexpr int kBvTrStride   = 68;                                 // floats per lane row of the transpose: 64 + 4 keeps 128-bit stores and
constexpr int kBvTrBytes    = 32 * kBvTrStride * 4;               // 64-bit loads free of bank conflicts
// per warp: the ring, the table slots, and the transpose buffer, which doubles as the dx staging area (6 x 512 bytes)
constexpr int kBvWarpBytes  = kBvStages * kBvStageBytes + kBvTabSlots * kBvTabBytes + kBvTrBytes;
constexpr int kBvSmem       = kWarpsPerCta * kBvWarpBytes;
static_assert(kBvSmem <= 227 * 1024, "one CTA per SM must fit");
static_assert(6 * kBvRowBytes <= kBvTrBytes, "dx staging fits the transpose buffer");

// Every node's table in the half-packed form of lut6_forward_keep_halves: 16 x (c[2k], c[2k+32], c[2k+1], c[2k+33]).
__global__ void __launch_bounds__(kWarpsPerCta * 32)
k_table_halves(const float *__restrict__ W, float4 *__restrict__ coef, int O, int lut_binarize)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int node = blockIdx.x * kWarpsPerCta + warp;
    if (node >= O) return;
    float2 v = reinterpret_cast<const float2 *>(W + (size_t)node * 64)[lane];
    if (lut_binarize) { v.x = v.x > 0.5f ? 1.0f : 0.0f; v.y = v.y > 0.5f ? 1.0f : 0.0f; }
    v = table_to_coeffs(v, lane);
    const float hx = __shfl_down_sync(kFull, v.x, 16), hy = __shfl_down_sync(kFull, v.y, 16);
    if (lane < 16) coef[(size_t)node * 16 + lane] = make_float4(v.x, hx, v.y, hy);
}

// dW += adjoint butterfly of the coefficient gradients (dC in the half-packed layout of k_table_halves); one warp per node.
__global__ void __launch_bounds__(kWarpsPerCta * 32)
k_coeff_grads_to_dw(const float4 *__restrict__ dC, float *__restrict__ dW, int O)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int node = blockIdx.x * kWarpsPerCta + warp;
    if (node >= O) return;
    const float4 e = dC[(size_t)node * 16 + (lane & 15)];
    const float2 g = lane < 16 ? make_float2(e.x, e.z) : make_float2(e.y, e.w);        // coefficients 2 lane, 2 lane + 1
    const float2 gw = coeff_grads_to_table(g, lane);
    float2 *dst = reinterpret_cast<float2 *>(dW + (size_t)node * 64) + lane;
    float2 cur = *dst;
    cur.x += gw.x; cur.y += gw.y;
    *dst = cur;
}

// The copies of input rows J..5 of a chunk: one shuffle and one 64-bit multiply-add per row, shared-memory offsets as immediates.
template <int J>
struct BvRowCopies {
    static __device__ __forceinline__ void issue(uint32_t sb, uint64_t gb, int row, uint64_t row_bytes)
    {
        cp_async16_at<J * kBvRowBytes, 0>(sb, gb + (uint64_t)__shfl_sync(0xffffffffu, row, J) * row_bytes);
        BvRowCopies<J + 1>::issue(sb, gb, row, row_bytes);
    }
};
template <>
struct BvRowCopies<6> {
    static __device__ __forceinline__ void issue(uint32_t, uint64_t, int, uint64_t) {}
};

// Position of a 128-frame chunk in a warp's sequence: item (tile, group), chunk c of the item's n, table slot of the item.
struct BvCursor {
    int tile, group, c, n, slot;
};

template <bool BN, bool BINARY>
__global__ void __launch_bounds__(kWarpsPerCta * 32, 1)
k_lut6_backward_pipe(const BwdArgs a, const float4 *__restrict__ coef, float *__restrict__ dC, int n_tiles, int n_full, int n_last)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char *my = smem_raw + (size_t)warp * kBvWarpBytes;
    unsigned char *my_tabs = my + kBvStages * kBvStageBytes;
    float *tr = reinterpret_cast<float *>(my_tabs + (kBvTabSlots * kBvTabBytes));

    const int step = (int)gridDim.x;
    const int dt = step / a.groups, dg = step - dt * a.groups;
    auto next_item = [&](BvCursor &p) {
        p.group += dg;
        p.tile += dt;
        if (p.group >= a.groups) { p.group -= a.groups; ++p.tile; }
        p.c = 0;
        p.n = p.tile == n_tiles - 1 ? n_last : n_full;
        p.slot = p.slot == kBvTabSlots - 1 ? 0 : p.slot + 1;
    };
    auto node_of = [&](const BvCursor &p) { return min(p.group * kWarpsPerCta + warp, a.O - 1); };      // a ragged last group repeats the last node
    auto row_of = [&](const BvCursor &p) { return (p.tile < n_tiles && lane < 6) ? __ldg(a.idx + (size_t)node_of(p) * 6 + lane) : 0; };

    BvCursor ic;
    ic.tile = (int)blockIdx.x / a.groups;
    ic.group = (int)blockIdx.x - ic.tile * a.groups;
    ic.c = 0;
    ic.n = ic.tile == n_tiles - 1 ? n_last : n_full;
    ic.slot = 0;
    BvCursor cc = ic;
    int ist = 0;
    int row_i = row_of(ic), row_in;
    {
        BvCursor t = ic;
        next_item(t);
        row_in = row_of(t);
    }
    const float *xf = static_cast<const float *>(a.x);
    const uint64_t x_global = (uint64_t)__cvta_generic_to_global(xf), dy_global = (uint64_t)__cvta_generic_to_global(a.dy);
    const uint64_t row_bytes = (uint64_t)a.xs * 4;
    auto issue = [&]() {
        if (ic.tile < n_tiles) {
            const int fc = ic.tile * a.T + ic.c * kFramesPerIter;              // first frame of the chunk
            const int f = fc + 4 * lane;
            unsigned char *st = my + ist * kBvStageBytes + lane * 16;
            const int node = node_of(ic);
            if (fc + kFramesPerIter <= a.xs && fc + kFramesPerIter <= a.dys) {
                // the whole chunk lies inside the rows (all but a last one): one 64-bit multiply-add per row, offsets as immediates
                const uint32_t sb = smem_addr(st);
                BvRowCopies<0>::issue(sb, x_global + (uint64_t)f * 4, row_i, row_bytes);
                cp_async16_at<6 * kBvRowBytes, 0>(sb, dy_global + ((uint64_t)node * (uint64_t)a.dys + (uint64_t)f) * 4);
            } else {
                const bool in_row = f < a.xs;
#pragma unroll
                for (int j = 0; j < 6; ++j) {
                    const int r = __shfl_sync(kFull, row_i, j);
                    cp_async16(st + j * kBvRowBytes, xf + (size_t)r * a.xs + (in_row ? f : 0), in_row);
                }
                cp_async16(st + 6 * kBvRowBytes, a.dy + (size_t)node * a.dys + (f < a.dys ? f : 0), f < a.dys);
            }
            if (ic.c == 0 && lane < 16) cp_async16(my_tabs + ic.slot * kBvTabBytes + lane * 16, coef + (size_t)node * 16 + lane, true);
            if (++ic.c == ic.n) {
                next_item(ic);
                row_i = row_in;
                BvCursor t = ic;
                next_item(t);
                row_in = row_of(t);
            }
        }
        cp_async_commit();
        ist = ist == kBvStages - 1 ? 0 : ist + 1;
    };
#pragma unroll
    for (int k = 0; k < kBvStages - 1; ++k) issue();

    int cst = 0;
    int row_c = row_of(cc), row_cn;
    float mean_n = 0.0f, rstd_n = 0.0f, dmean_n = 0.0f, dvar_n = 0.0f;
    if (BN && cc.tile < n_tiles) {
        const int n0 = node_of(cc);
        mean_n = a.mean[n0]; rstd_n = a.rstd[n0]; dmean_n = a.dmean[n0]; dvar_n = a.dvar[n0];
    }
    f32x2 acc2[32];
    while (cc.tile < n_tiles) {
        const int node_raw = cc.group * kWarpsPerCta + warp;
        const bool live_node = node_raw < a.O;
        const int node = min(node_raw, a.O - 1);
        const float mean = mean_n, rstd = rstd_n, dmean = dmean_n, dvar = dvar_n;
        {
            BvCursor t = cc;
            next_item(t);
            row_cn = row_of(t);
            if (BN && t.tile < n_tiles) {
                const int n1 = node_of(t);
                mean_n = a.mean[n1]; rstd_n = a.rstd[n1]; dmean_n = a.dmean[n1]; dvar_n = a.dvar[n1];
            }
        }
        const float4 *tab = reinterpret_cast<const float4 *>(my_tabs + cc.slot * kBvTabBytes);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc2[i] = 0ull;
        const int f_tile = cc.tile * a.T;
        for (; cc.c < cc.n; ++cc.c) {
            issue();                                 // refills the stage read kBvStages - 1 chunks ago (all lanes are past the barrier below)
            cp_async_wait<kBvStages - 1>();
            __syncwarp();                            // every lane's part of chunk k (and of this item's table) has landed
            const float *st2 = reinterpret_cast<const float *>(my + cst * kBvStageBytes) + 2 * lane;
            cst = cst == kBvStages - 1 ? 0 : cst + 1;
            const int f0 = f_tile + cc.c * kFramesPerIter;
            // lane l takes the frame pairs 64 h + 2 l + {0, 1}, h = 0, 1: one 64-bit shared load per row and pair, one 64-bit store per
            // input gradient and pair (both conflict-free)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float2 xp[6];
#pragma unroll
                for (int j = 0; j < 6; ++j) xp[j] = *reinterpret_cast<const float2 *>(st2 + j * kFramesPerIter + 64 * h);
                const float2 gp = *reinterpret_cast<const float2 *>(st2 + 6 * kFramesPerIter + 64 * h);
                float dxp[6][2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float u[6];
#pragma unroll
                    for (int j = 0; j < 6; ++j) {
                        const float v = e ? xp[j].y : xp[j].x;
                        u[j] = BINARY ? (v > 0.5f ? a.bias : -a.bias) : __saturatef(v) - 0.5f;           // the same values as condition_u()
                    }
                    KeptHalves D;
                    const float v = lut6_forward_keep_halves(tab, u, D);
                    float g = e ? gp.y : gp.x;
                    if (BN) {
                        const float tanh_x = ((v - mean) * rstd) * a.gamma + a.beta;
                        if (tanh_x <= 0.0f || tanh_x >= 1.0f) g = 0.0f;
                        const float dxc = (g * a.gamma) * rstd;
                        g = dxc + dmean + (v * dvar * a.rF);
                    }
                    if (f0 + 64 * h + 2 * lane + e >= a.F || !live_node) g = 0.0f;
                    float dxv[6];
                    lut6_reverse_halves(tab, u, D, g, acc2, dxv);
#pragma unroll
                    for (int j = 0; j < 6; ++j) dxp[j][e] = dxv[j];
                }
#pragma unroll
                for (int j = 0; j < 6; ++j) *reinterpret_cast<float2 *>(tr + j * kFramesPerIter + 64 * h + 2 * lane) = make_float2(dxp[j][0], dxp[j][1]);
            }
            __syncwarp();
            const bool write = f0 + 4 * lane < a.F && live_node;
#pragma unroll
            for (int j = 0; j < 6; ++j) {
                const int r = __shfl_sync(kFull, row_c, j);
                const float4 d = *reinterpret_cast<const float4 *>(tr + j * kFramesPerIter + 4 * lane);
                if (write) red_add_v4(a.dx + (size_t)r * a.dxs + f0 + 4 * lane, d.x, d.y, d.z, d.w);
            }
        }
        // ---- item done: sum the 64 accumulators over the lanes through the (padded) transpose
        __syncwarp();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float4 v;
            unpack2(acc2[2 * k], v.x, v.y);
            unpack2(acc2[2 * k + 1], v.z, v.w);
            *reinterpret_cast<float4 *>(tr + lane * kBvTrStride + 4 * k) = v;
        }
        __syncwarp();
        f32x2 s0 = 0ull, s1 = 0ull, s2 = 0ull, s3 = 0ull;
#pragma unroll
        for (int r = 0; r < 32; r += 4) {
            s0 = add2(s0, *reinterpret_cast<const f32x2 *>(tr + (r + 0) * kBvTrStride + 2 * lane));
            s1 = add2(s1, *reinterpret_cast<const f32x2 *>(tr + (r + 1) * kBvTrStride + 2 * lane));
            s2 = add2(s2, *reinterpret_cast<const f32x2 *>(tr + (r + 2) * kBvTrStride + 2 * lane));
            s3 = add2(s3, *reinterpret_cast<const f32x2 *>(tr + (r + 3) * kBvTrStride + 2 * lane));
        }
        float lo, hi;
        unpack2(add2(add2(s0, s1), add2(s2, s3)), lo, hi);
        if (live_node) red_add_v2(dC + (size_t)node * 64 + 2 * lane, lo, hi);
        __syncwarp();                                // the transpose buffer is the next chunk's dx staging area
        next_item(cc);
        row_c = row_cn;
    }
    cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------
static int check_common(const void *x, const void *y, const int *idx, const float *W, int O, int F, long long stride)
{
    BB200_REQUIRE_PTR(x); BB200_REQUIRE_PTR(y); BB200_REQUIRE_PTR(idx); BB200_REQUIRE_PTR(W);
    BB200_REQUIRE(O >= 0 && F >= 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE(stride >= 0, BBCU_ERR_BAD_STRIDE);
    BB200_REQUIRE((reinterpret_cast<uintptr_t>(W) & 7) == 0, BBCU_ERR_BAD_STRIDE);
    return BBCU_OK;
}

// opt-in to more than 48 KB of dynamic shared memory (per kernel and device; the call is a host-side attribute write)
template <typename K>
static bool allow_big_smem(K kernel, int bytes)
{
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) { cudaGetLastError(); return false; }
    return true;
}

template <bool XBIT, int PHASE, bool YBIT>
static int launch_forward(FwdArgs a, int max_tile, cudaStream_t st)
{
    if (a.O == 0 || a.F == 0) return BBCU_OK;
    a.groups = (a.O + kWarpsPerCta - 1) / kWarpsPerCta;
    // input count is not part of this ABI: between O (square layer) and 6*O rows are touched
    a.T = frame_tile(3LL * a.O, XBIT ? 1 : 32, a.groups, a.F, max_tile);
    if (!XBIT && !YBIT) {
        // pipelined path: rows and tables must start on 16-byte boundaries for the 16-byte copies and the 128-bit stores
        const bool aligned = ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.W) | reinterpret_cast<uintptr_t>(a.y)) & 15) == 0 &&
                             (a.xs % 4) == 0 && (a.ys % 4) == 0;
        auto kern = a.binary ? k_lut6_forward_pipe<PHASE, true> : k_lut6_forward_pipe<PHASE, false>;
        if (aligned && allow_big_smem(kern, kFpSmem)) {
            // 256-frame items whenever there are that many frames: four frame pairs per lane share every table read and the
            // per-item costs halve.  Measured on B200: 65536 -> 65536 nodes x 4096 frames 1.89 ms (128) vs 1.49 ms (256), although
            // the 256-frame tile of such a layer (64 MiB of gathered rows) no longer fits a fifth of L2.
            a.T = a.F > kFramesPerIter ? kFpMaxItemFrames : kFramesPerIter;
            const long long n_items = (long long)((a.F + a.T - 1) / a.T) * a.groups;
            BB200_REQUIRE(n_items < (1LL << 31) - 4096, BBCU_ERR_TOO_LARGE);      // 32-bit item arithmetic in the kernel
            long long grid = (long long)kFpCtas * device_info().sm_count;
            if (grid > n_items) grid = n_items;
            if (!a.no_scratch) {
                // slot 1 of the stream's scratch: slot 0 may hold the caller's batch-norm sums at the same time
                float4 *coef = static_cast<float4 *>(stream_scratch(st, (size_t)a.O * kFpTabSlotBytes, 1));
                if (coef != nullptr) {
                    k_table_coeffs<<<a.groups, kWarpsPerCta * 32, 0, st>>>(a.W, coef, a.O, a.lut_binarize);
                    BB200_CUDA(cudaPeekAtLastError());
                    a.coef = coef;
                }
            }
            kern<<<(unsigned)grid, kWarpsPerCta * 32, kFpSmem, st>>>(a, (a.F + a.T - 1) / a.T);
            return launch_status();
        }
    }
    const long long tiles = (a.F + a.T - 1) / a.T;
    const long long blocks = tiles * a.groups;
    BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
    k_lut6_forward<XBIT, PHASE, YBIT><<<(unsigned)blocks, kWarpsPerCta * 32, 0, st>>>(a);
    return launch_status();
}

// The statistics half of the fp32 backward (the two batch-norm sums from a re-evaluated LUT value and dy) through the pipelined
// forward kernel, which evaluates the tree at nearly twice the rate of k_lut6_backward_stats.  Returns false, having launched
// nothing, when the rows are not 16-byte aligned or the shared-memory opt-in is refused; *rc is the launch status otherwise.
// b.sums must be zero on entry.
static bool backward_stats_pipe(const BwdArgs &b, cudaStream_t st, int *rc, void *tmp = nullptr, size_t tmp_bytes = 0)
{
    const bool aligned = ((reinterpret_cast<uintptr_t>(b.x) | reinterpret_cast<uintptr_t>(b.W) | reinterpret_cast<uintptr_t>(b.dy)) & 15) == 0 &&
                         (b.xs % 4) == 0 && (b.dys % 4) == 0;
    auto kern = b.binary ? k_lut6_forward_pipe<PH_BWD, true> : k_lut6_forward_pipe<PH_BWD, false>;
    if (!aligned || !allow_big_smem(kern, kFpSmem)) return false;
    FwdArgs a = {};
    a.x = b.x; a.idx = b.idx; a.W = b.W; a.mean = b.mean; a.rstd = b.rstd; a.sums = b.sums; a.dy = b.dy; a.dys = b.dys;
    a.gamma = b.gamma; a.beta = b.beta; a.bias = b.bias;
    a.O = b.O; a.F = b.F; a.xs = b.xs; a.ys = b.xs; a.lut_binarize = b.lut_binarize; a.binary = b.binary;
    a.groups = (a.O + kWarpsPerCta - 1) / kWarpsPerCta;
    a.T = a.F > kFramesPerIter ? kFpMaxItemFrames : kFramesPerIter;
    const long long n_items = (long long)((a.F + a.T - 1) / a.T) * a.groups;
    if (n_items >= (1LL << 31) - 4096) return false;
    long long grid = (long long)kFpCtas * device_info().sm_count;
    if (grid > n_items) grid = n_items;
    // converted tables: the caller's scratch when it is large enough (the backward proper reuses it afterwards, in stream order),
    // else slot 1 of the stream's scratch; without either the kernel converts the raw tables itself
    const size_t need = (size_t)a.O * kFpTabSlotBytes;
    float4 *coef = (tmp != nullptr && tmp_bytes >= need && (reinterpret_cast<uintptr_t>(tmp) & 15) == 0)
                       ? static_cast<float4 *>(tmp) : static_cast<float4 *>(stream_scratch(st, need, 1));
    if (coef != nullptr) {
        k_table_coeffs<<<a.groups, kWarpsPerCta * 32, 0, st>>>(a.W, coef, a.O, a.lut_binarize);
        a.coef = coef;
    }
    kern<<<(unsigned)grid, kWarpsPerCta * 32, kFpSmem, st>>>(a, (a.F + a.T - 1) / a.T);
    *rc = launch_status();
    return true;
}

template <bool XBIT>
static int forward_plain(const void *x, float *y, uint32_t *ybits, const int *idx, const float *W, int O, int F, long long xs, long long ys,
                         int binary, int lut_binarize, float bias, cudaStream_t st)
{
    FwdArgs a = {};
    a.x = x; a.y = y; a.ybits = ybits; a.idx = idx; a.W = W; a.bias = bias;
    a.O = O; a.F = F; a.xs = xs; a.ys = ys; a.lut_binarize = lut_binarize; a.binary = binary;
    if (ybits) return launch_forward<XBIT, PH_PLAIN, true>(a, 2048, st);
    return launch_forward<XBIT, PH_PLAIN, false>(a, 2048, st);
}

// Frames per tile of the persistent backward.  A wide tile amortises the per-item flush of the 64 gradient sums; a narrow one keeps
// the tile's x and dx rows (8 bytes per row and frame) in L2.  The kernel is issue-bound, so the wide tile wins until the rows
// exceed L2 several times over -- measured on B200: 8192 rows 1.60 / 1.54 / 1.52 ms at 512 / 1024 / 2048 frames, 65536 rows
// 3.57 / 3.42 / 3.46 ms -- hence four times L2, between 512 and 2048 frames.
static int backward_pipe_tile(long long rows, int groups, int F)
{
    const DeviceInfo &di = device_info();
    long long t = (long long)(4 * di.l2_bytes) / (8 * (rows > 0 ? rows : 1));
    t = (t / kFramesPerIter) * kFramesPerIter;
    if (t > 2048) t = 2048;
    if (t < 512) t = 512;
    // small layers: narrow the tile until every SM has a couple of items
    while (t > kFramesPerIter && (long long)groups * ((F + t - 1) / t) < 2LL * di.sm_count) t -= kFramesPerIter;
    return (int)t;
}

// The persistent backward (k_lut6_backward_pipe); BBCU_ERR_NO_MEMORY when its scratch (512 bytes per node) cannot be had.
// `tmp` / `tmp_bytes`: scratch handed in by the caller (the reference's dev_dx_tmp), used when it is large enough and 16-byte aligned.
static int launch_backward_pipe(BwdArgs a, bool bn, int I, void *tmp, size_t tmp_bytes, cudaStream_t st)
{
    const size_t need = (size_t)a.O * 512;
    unsigned char *scratch = nullptr;
    if (tmp != nullptr && tmp_bytes >= need && (reinterpret_cast<uintptr_t>(tmp) & 15) == 0) scratch = static_cast<unsigned char *>(tmp);
    else scratch = static_cast<unsigned char *>(stream_scratch(st, need, 1));
    if (scratch == nullptr) return BBCU_ERR_NO_MEMORY;
    float4 *coef = reinterpret_cast<float4 *>(scratch);
    float *dC = reinterpret_cast<float *>(scratch + (size_t)a.O * 256);
    auto kern = bn ? (a.binary ? k_lut6_backward_pipe<true, true> : k_lut6_backward_pipe<true, false>)
                   : (a.binary ? k_lut6_backward_pipe<false, true> : k_lut6_backward_pipe<false, false>);
    if (!allow_big_smem(kern, kBvSmem)) return BBCU_ERR_NO_MEMORY;
    const long long rows = (long long)(I < 6LL * a.O ? I : 6LL * a.O);
    a.T = backward_pipe_tile(rows, a.groups, a.F);
    const int n_tiles = (a.F + a.T - 1) / a.T;
    const long long n_items = (long long)n_tiles * a.groups;
    BB200_REQUIRE(n_items < (1LL << 31) - 4096, BBCU_ERR_TOO_LARGE);          // 32-bit item arithmetic in the kernel
    const int n_full = a.T / kFramesPerIter;
    const int n_last = (a.F - (n_tiles - 1) * a.T + kFramesPerIter - 1) / kFramesPerIter;
    long long grid = device_info().sm_count;
    if (grid > n_items) grid = n_items;
    const int groups8 = (a.O + kWarpsPerCta - 1) / kWarpsPerCta;
    k_table_halves<<<groups8, kWarpsPerCta * 32, 0, st>>>(a.W, coef, a.O, a.lut_binarize);
    BB200_CUDA(cudaPeekAtLastError());
    BB200_CUDA(cudaMemsetAsync(dC, 0, (size_t)a.O * 256, st));
    kern<<<(unsigned)grid, kWarpsPerCta * 32, kBvSmem, st>>>(a, coef, dC, n_tiles, n_full, n_last);
    BB200_CUDA(cudaPeekAtLastError());
    k_coeff_grads_to_dw<<<groups8, kWarpsPerCta * 32, 0, st>>>(reinterpret_cast<const float4 *>(dC), a.dW, a.O);
    return launch_status();
}

// Zero fill with 128-bit stores from a grid sized to the GPU.  A large cudaMemsetAsync ran at about half of the copy bandwidth
// (8 GiB of dx in 2.7 ms); the clear is 6 % of a training step, so it gets a kernel.
__global__ void __launch_bounds__(256)
k_zero_fill(float4 *__restrict__ p, size_t n)
{
    const float4 z = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = z;
}

static int zero_async(void *ptr, size_t bytes, cudaStream_t st)
{
    if (bytes >= ((size_t)1 << 20) && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0) {
        const size_t n = bytes / 16;
        k_zero_fill<<<(unsigned)(8 * device_info().sm_count), 256, 0, st>>>(static_cast<float4 *>(ptr), n);
        BB200_CUDA(cudaPeekAtLastError());
        if (bytes % 16) BB200_CUDA(cudaMemsetAsync(static_cast<unsigned char *>(ptr) + n * 16, 0, bytes % 16, st));
        return BBCU_OK;
    }
    BB200_CUDA(cudaMemsetAsync(ptr, 0, bytes, st));
    return BBCU_OK;
}

template <bool XBIT>
static int backward_common(BwdArgs a, bool bn, long long total_frames, float *dmean_out, float *dvar_out, const double *ext_sums,
                           int I, cudaStream_t st, void *tmp = nullptr, size_t tmp_bytes = 0)
{
    // dx starts from zero (the reference's CPU path: dx_buf.FillZero(), DifferentiableLutN.h:1159)
    if (I > 0 && a.dxs > 0) {
        const int rc = zero_async(a.dx, sizeof(float) * (size_t)I * a.dxs, st);
        if (rc) return rc;
    }
    if (a.O == 0 || a.F == 0) return BBCU_OK;
    if ((XBIT || a.binary) && ext_sums == nullptr && a.dys == a.dxs && total_frames == a.F) {
        // two-valued inputs (bit frames, or fp32 frames in binary mode): everything factors through the 6-bit input pattern of a
        // frame (binary_mode.cu)
        const int rc = bit_backward_by_table(bn, !XBIT, a.x, a.dy, a.dx, a.idx, a.W, a.dW, a.mean, a.rstd, dmean_out, dvar_out, a.gamma, a.beta,
                                             a.bias, a.O, a.F, a.xs, a.dxs, a.lut_binarize, st);
        if (rc != BBCU_ERR_NO_MEMORY) return rc;
    }
    if ((XBIT || a.binary) && bn && ext_sums != nullptr && a.dys == a.dxs) {
        // frame-sharded caller: the apply half of the same route, with the batch sums of all ranks
        const int rc = bit_backward_apply_by_table(!XBIT, a.x, a.dy, a.dx, a.idx, a.W, a.dW, a.mean, a.rstd, ext_sums, dmean_out, dvar_out, a.gamma,
                                                   a.beta, a.bias, a.O, a.F, a.xs, a.dxs, total_frames, a.lut_binarize, st);
        if (rc != BBCU_ERR_NO_MEMORY) return rc;
    }
    a.groups = (a.O + kWarpsPerCta - 1) / kWarpsPerCta;
    const long long rows = (long long)(I < 6LL * a.O ? I : 6LL * a.O);
    // Wide tiles: a warp reduces its 64 dW accumulators across lanes once per (node, tile), about 250 instructions, so the
    // tile is made as wide as still leaves two CTAs per SM.  Measured on B200 (65536 -> 65536 nodes, 4096 frames): 7.9 ms
    // with L2-sized 128-frame tiles, 5.2 ms with 4096-frame tiles -- the extra L2 misses cost less than the reductions.
    (void)rows;
    a.T = 4096;          // 2048 / 1024 / 512 measured 4 % / 8 % / 18 % slower on the 8192-node layer with the current kernel
    while (a.T > kFramesPerIter && (long long)a.groups * ((a.F + a.T - 1) / a.T) < 2LL * device_info().sm_count) a.T /= 2;
    const long long tiles = (a.F + a.T - 1) / a.T;
    const long long blocks = tiles * a.groups;
    BB200_REQUIRE(blocks < (1LL << 31) - 4096, BBCU_ERR_TOO_LARGE);
    a.rF = 1.0f / (float)total_frames;
    if (bn) {
        if (ext_sums == nullptr) {
            double *sums = static_cast<double *>(stream_scratch(st, sizeof(double) * 2 * (size_t)a.O));
            BB200_REQUIRE(sums != nullptr, BBCU_ERR_NO_MEMORY);
            BB200_CUDA(cudaMemsetAsync(sums, 0, sizeof(double) * 2 * (size_t)a.O, st));
            a.sums = sums;
            int rc = BBCU_OK;
            if (XBIT || !backward_stats_pipe(a, st, &rc, tmp, tmp_bytes)) {
                k_lut6_backward_stats<XBIT><<<(unsigned)blocks, kWarpsPerCta * 32, 0, st>>>(a);
                rc = launch_status();
            }
            if (rc) return rc;
            ext_sums = sums;
        }
        k_bn_backward_finalize<<<(a.O + 255) / 256, 256, 0, st>>>(ext_sums, a.mean, a.rstd, dmean_out, dvar_out, a.O, total_frames);
        BB200_CUDA(cudaPeekAtLastError());
        a.dmean = dmean_out; a.dvar = dvar_out;
    }
    if (!XBIT) {
        // rows on 16-byte boundaries (the FrameBuffer layout gives them): the persistent kernel
        const bool aligned = ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.dy) | reinterpret_cast<uintptr_t>(a.dx) |
                               reinterpret_cast<uintptr_t>(a.dW)) & 15) == 0 && (a.xs % 4) == 0 && (a.dys % 4) == 0 && (a.dxs % 4) == 0;
        if (aligned) {
            const int rc = launch_backward_pipe(a, bn, I, tmp, tmp_bytes, st);
            if (rc != BBCU_ERR_NO_MEMORY) return rc;
        }
    }
    if (bn) k_lut6_backward<XBIT, true><<<(unsigned)blocks, kWarpsPerCta * 32, 0, st>>>(a);
    else    k_lut6_backward<XBIT, false><<<(unsigned)blocks, kWarpsPerCta * 32, 0, st>>>(a);
    return launch_status();
}

}   // namespace bb200

using namespace bb200;

// Bytes of the caller's dx_tmp buffer: the reference allocates it as output_node_size * 6 rows of tmp_frame_stride floats
// (include/bb/DifferentiableLutN.h:1038-1042).
static size_t dx_tmp_bytes(const void *dx_tmp, int output_node_size, int tmp_frame_stride)
{
    if (dx_tmp == nullptr || output_node_size <= 0 || tmp_frame_stride <= 0) return 0;
    return (size_t)output_node_size * 6 * (size_t)tmp_frame_stride * sizeof(float);
}

// ------------------------------------------------------------------------------------------- StochasticLut6
extern "C" int bbcu_fp32_StochasticLut6_Forward(const float *x, float *y, const int *idx, const float *W, int node_size, int frame_size,
                                                int frame_stride, int input_binary, int lut_binarize, float unbinarize_bias, bbcu_stream_t stream)
{
    int rc = check_common(x, y, idx, W, node_size, frame_size, frame_stride);
    if (rc) return rc;
    BB200_REQUIRE(frame_stride >= frame_size, BBCU_ERR_BAD_STRIDE);
    if (input_binary) {       // two-valued inputs: per-pattern values, looked up per frame (binary_mode.cu)
        rc = f32_binary_forward_by_table(0, x, y, idx, W, nullptr, nullptr, nullptr, nullptr, 0.0f, 0.0f, 0.0f, unbinarize_bias, node_size, frame_size,
                                         frame_stride, lut_binarize, as_stream(stream));
        if (rc != BBCU_ERR_NO_MEMORY) return rc;
    }
    return forward_plain<false>(x, y, nullptr, idx, W, node_size, frame_size, frame_stride, frame_stride, input_binary, lut_binarize,
                                unbinarize_bias, as_stream(stream));
}

extern "C" int bbcu_bit_fp32_StochasticLut6_Forward(const int *x, float *y, const int *idx, const float *W, int node_size, int frame_size,
                                                    int frame_stride, int bin_frame_stride, int lut_binarize, float unbinarize_bias,
                                                    bbcu_stream_t stream)
{
    int rc = check_common(x, y, idx, W, node_size, frame_size, frame_stride);
    if (rc) return rc;
    BB200_REQUIRE(frame_stride >= frame_size && (long long)bin_frame_stride * 32 >= frame_size, BBCU_ERR_BAD_STRIDE);
    // bit inputs: the node's value is one of 64 per-pattern values, looked up per frame
    rc = bit_fp32_forward_by_table(x, y, idx, W, unbinarize_bias, node_size, frame_size, bin_frame_stride, frame_stride, lut_binarize,
                                   as_stream(stream));
    if (rc != BBCU_ERR_NO_MEMORY) return rc;
    return forward_plain<true>(x, y, nullptr, idx, W, node_size, frame_size, bin_frame_stride, frame_stride, 1, lut_binarize,
                               unbinarize_bias, as_stream(stream));
}

extern "C" int bbcu_bit_bit_fp32_StochasticLut6_Forward(const int *x, int *y, const int *idx, const float *W, int node_size, int frame_size,
                                                        int frame_stride, int lut_binarize, float unbinarize_bias, bbcu_stream_t stream)
{
    int rc = check_common(x, y, idx, W, node_size, frame_size, frame_stride);
    if (rc) return rc;
    BB200_REQUIRE((long long)frame_stride * 32 >= frame_size, BBCU_ERR_BAD_STRIDE);
    // bit in, bit out: the layer is a BinaryLut6 forward with the truth table (LUT value of each input pattern > 0.5)
    rc = bit_forward_by_table(false, x, y, idx, W, nullptr, nullptr, 0.0f, 0.0f, unbinarize_bias, node_size, frame_size, frame_stride,
                              lut_binarize, as_stream(stream));
    if (rc != BBCU_ERR_NO_MEMORY) return rc;
    return forward_plain<true>(x, nullptr, reinterpret_cast<uint32_t *>(y), idx, W, node_size, frame_size, frame_stride, frame_stride, 1,
                               lut_binarize, unbinarize_bias, as_stream(stream));
}

extern "C" int bbcu_fp32_StochasticLut6_Backward(const float *x, const float *dy, float *dx, float *dx_tmp, const int *idx, const int *rev,
                                                 const float *W, float *dW, int reverse_index_stride, int input_node_size, int output_node_size,
                                                 int frame_size, int frame_stride, int tmp_frame_size, int tmp_frame_stride,
                                                 int input_binary, int lut_binarize, float unbinarize_bias, bbcu_stream_t stream)
{
    (void)rev; (void)reverse_index_stride; (void)tmp_frame_size;
    int rc = check_common(x, dx, idx, W, output_node_size, frame_size, frame_stride);
    if (rc) return rc;
    BB200_REQUIRE_PTR(dy); BB200_REQUIRE_PTR(dW);
    BB200_REQUIRE(input_node_size >= 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE(frame_stride >= frame_size, BBCU_ERR_BAD_STRIDE);
    BwdArgs a = {};
    a.x = x; a.dy = dy; a.dx = dx; a.idx = idx; a.W = W; a.dW = dW; a.bias = unbinarize_bias;
    a.O = output_node_size; a.F = frame_size; a.xs = frame_stride; a.dys = frame_stride; a.dxs = frame_stride;
    a.lut_binarize = lut_binarize; a.binary = input_binary;
    return backward_common<false>(a, false, frame_size > 0 ? frame_size : 1, nullptr, nullptr, nullptr, input_node_size, as_stream(stream),
                                  dx_tmp, dx_tmp_bytes(dx_tmp, output_node_size, tmp_frame_stride));
}

extern "C" int bbcu_bit_fp32_StochasticLut6_Backward(const int *x, const float *dy, float *dx, float *dx_tmp, const int *idx, const int *rev,
                                                     const float *W, float *dW, int reverse_index_stride, int input_node_size,
                                                     int output_node_size, int frame_size, int frame_stride, int bin_frame_stride,
                                                     int tmp_frame_size, int tmp_frame_stride, int lut_binarize, float unbinarize_bias,
                                                     bbcu_stream_t stream)
{
    (void)dx_tmp; (void)rev; (void)reverse_index_stride; (void)tmp_frame_size; (void)tmp_frame_stride;
    int rc = check_common(x, dx, idx, W, output_node_size, frame_size, frame_stride);
    if (rc) return rc;
    BB200_REQUIRE_PTR(dy); BB200_REQUIRE_PTR(dW);
    BB200_REQUIRE(input_node_size >= 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE(frame_stride >= frame_size && (long long)bin_frame_stride * 32 >= frame_size, BBCU_ERR_BAD_STRIDE);
    BwdArgs a = {};
    a.x = x; a.dy = dy; a.dx = dx; a.idx = idx; a.W = W; a.dW = dW; a.bias = unbinarize_bias;
    a.O = output_node_size; a.F = frame_size; a.xs = bin_frame_stride; a.dys = frame_stride; a.dxs = frame_stride;
    a.lut_binarize = lut_binarize; a.binary = 1;
    return backward_common<true>(a, false, frame_size > 0 ? frame_size : 1, nullptr, nullptr, nullptr, input_node_size, as_stream(stream));
}

// ------------------------------------------------------------------------------------------- DifferentiableLut6
static int dl6_finalize_and_normalize(float *y, const double *sums, float *mean, float *rstd, float *rmean, float *rvar,
                                      float gamma, float beta, float momentum, int O, int F, long long ys, long long total_frames,
                                      int binary, cudaStream_t st)
{
    if (O == 0) return BBCU_OK;
    k_bn_finalize<<<(O + 255) / 256, 256, 0, st>>>(sums, mean, rstd, rmean, rvar, momentum, O, total_frames);
    BB200_CUDA(cudaPeekAtLastError());
    if (y != nullptr && F > 0) {
        const int chunks = (F + 4095) / 4096;
        const long long blocks = (long long)O * chunks;
        BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
        k_bn_normalize_inplace<<<(unsigned)blocks, 256, 0, st>>>(y, mean, rstd, gamma, beta, F, ys, binary, chunks);
    }
    return launch_status();
}

namespace bb200 {
int dl6_forward_stats(const float *x, float *y, const int *idx, const float *W, double *dev_sums, float unbinarize_bias, int node_size,
                      int frame_size, int frame_stride, int lut_binarize, int binary_mode, bool may_allocate, cudaStream_t st)
{
    int rc = check_common(x, y, idx, W, node_size, frame_size, frame_stride);
    if (rc) return rc;
    BB200_REQUIRE_PTR(dev_sums);
    BB200_REQUIRE(frame_stride >= frame_size, BBCU_ERR_BAD_STRIDE);
    if (binary_mode && may_allocate) {       // two-valued inputs: raw values by per-pattern lookup, sums from the pattern counts
        rc = f32_binary_forward_by_table(3, x, y, idx, W, reinterpret_cast<float *>(dev_sums), nullptr, nullptr, nullptr, 0.0f, 0.0f, 0.0f,
                                         unbinarize_bias, node_size, frame_size, frame_stride, lut_binarize, st);
        if (rc != BBCU_ERR_NO_MEMORY) return rc;
    }
    BB200_CUDA(cudaMemsetAsync(dev_sums, 0, sizeof(double) * 2 * (size_t)node_size, st));
    FwdArgs a = {};
    a.x = x; a.y = y; a.idx = idx; a.W = W; a.sums = dev_sums; a.bias = unbinarize_bias;
    a.O = node_size; a.F = frame_size; a.xs = frame_stride; a.ys = frame_stride; a.lut_binarize = lut_binarize; a.binary = binary_mode;
    a.no_scratch = may_allocate ? 0 : 1;
    return launch_forward<false, PH_STATS, false>(a, 2048, st);
}
}   // namespace bb200

extern "C" int bbcu_fp32_DifferentiableLut6_ForwardStats(const float *x, float *y, const int *idx, const float *W, double *dev_sums,
                                                         float unbinarize_bias, int node_size, int frame_size, int frame_stride,
                                                         int lut_binarize, int binary_mode, bbcu_stream_t stream)
{
    return dl6_forward_stats(x, y, idx, W, dev_sums, unbinarize_bias, node_size, frame_size, frame_stride, lut_binarize, binary_mode, true,
                             as_stream(stream));
}

extern "C" int bbcu_fp32_DifferentiableLut6_ForwardNormalize(float *y, const double *dev_sums, float *mean, float *rstd, float *rmean,
                                                             float *rvar, float gamma, float beta, float momentum, int node_size,
                                                             int frame_size, int frame_stride, long long total_frame_size, int binary_mode,
                                                             bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(y); BB200_REQUIRE_PTR(dev_sums); BB200_REQUIRE_PTR(mean); BB200_REQUIRE_PTR(rstd); BB200_REQUIRE_PTR(rmean); BB200_REQUIRE_PTR(rvar);
    BB200_REQUIRE(node_size >= 0 && frame_size >= 0 && total_frame_size >= frame_size && total_frame_size > 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE(frame_stride >= frame_size, BBCU_ERR_BAD_STRIDE);
    return dl6_finalize_and_normalize(y, dev_sums, mean, rstd, rmean, rvar, gamma, beta, momentum, node_size, frame_size, frame_stride,
                                      total_frame_size, binary_mode, as_stream(stream));
}

extern "C" int bbcu_fp32_DifferentiableLut6_ForwardTraining(const float *x, float *y, const int *idx, const float *W, float *mean, float *rstd,
                                                            float *rmean, float *rvar, float gamma, float beta, float momentum,
                                                            float unbinarize_bias, int node_size, int frame_size, int frame_stride,
                                                            int lut_binarize, int binary_mode, bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(mean); BB200_REQUIRE_PTR(rstd); BB200_REQUIRE_PTR(rmean); BB200_REQUIRE_PTR(rvar);
    BB200_REQUIRE(frame_size > 0 || node_size == 0, BBCU_ERR_BAD_SIZE);
    if (node_size == 0) return BBCU_OK;
    cudaStream_t st = as_stream(stream);
    if (binary_mode) {        // two-valued inputs, binarised output: statistics from the pattern counts, output from the truth table
        int rcb = check_common(x, y, idx, W, node_size, frame_size, frame_stride);
        if (rcb) return rcb;
        BB200_REQUIRE(frame_stride >= frame_size, BBCU_ERR_BAD_STRIDE);
        rcb = f32_binary_forward_by_table(2, x, y, idx, W, mean, rstd, rmean, rvar, gamma, beta, momentum, unbinarize_bias, node_size, frame_size,
                                          frame_stride, lut_binarize, st);
        if (rcb != BBCU_ERR_NO_MEMORY) return rcb;
    }
    double *sums = static_cast<double *>(stream_scratch(st, sizeof(double) * 2 * (size_t)(node_size > 0 ? node_size : 0)));
    BB200_REQUIRE(sums != nullptr, BBCU_ERR_NO_MEMORY);
    int rc = bbcu_fp32_DifferentiableLut6_ForwardStats(x, y, idx, W, sums, unbinarize_bias, node_size, frame_size, frame_stride, lut_binarize,
                                                       binary_mode, stream);
    if (rc) return rc;
    return dl6_finalize_and_normalize(y, sums, mean, rstd, rmean, rvar, gamma, beta, momentum, node_size, frame_size, frame_stride, frame_size,
                                      binary_mode, st);
}

extern "C" int bbcu_bit_fp32_DifferentiableLut6_ForwardTraining(const int *x, int *y, const int *idx, const float *W, float *mean, float *rstd,
                                                                float *rmean, float *rvar, float gamma, float beta, float momentum,
                                                                float unbinarize_bias, int node_size, int frame_size, int frame_stride,
                                                                int lut_binarize, bbcu_stream_t stream)
{
    int rc = check_common(x, y, idx, W, node_size, frame_size, frame_stride);
    if (rc) return rc;
    BB200_REQUIRE_PTR(mean); BB200_REQUIRE_PTR(rstd); BB200_REQUIRE_PTR(rmean); BB200_REQUIRE_PTR(rvar);
    BB200_REQUIRE(frame_size > 0 || node_size == 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE((long long)frame_stride * 32 >= frame_size, BBCU_ERR_BAD_STRIDE);
    if (node_size == 0) return BBCU_OK;
    cudaStream_t st = as_stream(stream);
    // bit in, bit out: statistics from the per-node histogram of input patterns, output by a BinaryLut6 forward with the truth table
    rc = dl6_bit_forward_training_by_table(x, y, idx, W, mean, rstd, rmean, rvar, gamma, beta, momentum, unbinarize_bias, node_size, frame_size,
                                           frame_stride, lut_binarize, st);
    if (rc != BBCU_ERR_NO_MEMORY) return rc;
    double *sums = static_cast<double *>(stream_scratch(st, sizeof(double) * 2 * (size_t)node_size));
    BB200_REQUIRE(sums != nullptr, BBCU_ERR_NO_MEMORY);
    BB200_CUDA(cudaMemsetAsync(sums, 0, sizeof(double) * 2 * (size_t)node_size, st));
    FwdArgs a = {};
    a.x = x; a.ybits = reinterpret_cast<uint32_t *>(y); a.idx = idx; a.W = W; a.sums = sums; a.bias = unbinarize_bias;
    a.gamma = gamma; a.beta = beta;
    a.O = node_size; a.F = frame_size; a.xs = frame_stride; a.ys = frame_stride; a.lut_binarize = lut_binarize; a.binary = 1;
    rc = launch_forward<true, PH_STATS, true>(a, 2048, st);
    if (rc) return rc;
    rc = dl6_finalize_and_normalize(nullptr, sums, mean, rstd, rmean, rvar, gamma, beta, momentum, node_size, frame_size, frame_stride,
                                    frame_size, 1, st);
    if (rc) return rc;
    a.mean = mean; a.rstd = rstd; a.stat_is_var = 0;
    return launch_forward<true, PH_NORM, true>(a, 2048, st);
}

extern "C" int bbcu_fp32_DifferentiableLut6_ForwardInference(const float *x, float *y, const int *idx, const float *W, const float *rmean,
                                                             const float *rvar, float gamma, float beta, float unbinarize_bias, int node_size,
                                                             int frame_size, int frame_stride, int lut_binarize, int binary_mode,
                                                             bbcu_stream_t stream)
{
    int rc = check_common(x, y, idx, W, node_size, frame_size, frame_stride);
    if (rc) return rc;
    BB200_REQUIRE_PTR(rmean); BB200_REQUIRE_PTR(rvar);
    BB200_REQUIRE(frame_stride >= frame_size, BBCU_ERR_BAD_STRIDE);
    if (binary_mode) {
        rc = f32_binary_forward_by_table(1, x, y, idx, W, nullptr, nullptr, const_cast<float *>(rmean), const_cast<float *>(rvar), gamma, beta, 0.0f,
                                         unbinarize_bias, node_size, frame_size, frame_stride, lut_binarize, as_stream(stream));
        if (rc != BBCU_ERR_NO_MEMORY) return rc;
    }
    FwdArgs a = {};
    a.x = x; a.y = y; a.idx = idx; a.W = W; a.mean = rmean; a.rstd = rvar; a.stat_is_var = 1; a.bias = unbinarize_bias;
    a.gamma = gamma; a.beta = beta;
    a.O = node_size; a.F = frame_size; a.xs = frame_stride; a.ys = frame_stride; a.lut_binarize = lut_binarize; a.binary = binary_mode;
    return launch_forward<false, PH_NORM, false>(a, 2048, as_stream(stream));
}

extern "C" int bbcu_bit_fp32_DifferentiableLut6_ForwardInference(const int *x, int *y, const int *idx, const float *W, const float *rmean,
                                                                 const float *rvar, float gamma, float beta, float unbinarize_bias,
                                                                 int node_size, int frame_size, int frame_stride, int lut_binarize,
                                                                 bbcu_stream_t stream)
{
    int rc = check_common(x, y, idx, W, node_size, frame_size, frame_stride);
    if (rc) return rc;
    BB200_REQUIRE_PTR(rmean); BB200_REQUIRE_PTR(rvar);
    BB200_REQUIRE((long long)frame_stride * 32 >= frame_size, BBCU_ERR_BAD_STRIDE);
    rc = bit_forward_by_table(true, x, y, idx, W, rmean, rvar, gamma, beta, unbinarize_bias, node_size, frame_size, frame_stride, lut_binarize,
                              as_stream(stream));
    if (rc != BBCU_ERR_NO_MEMORY) return rc;
    FwdArgs a = {};
    a.x = x; a.ybits = reinterpret_cast<uint32_t *>(y); a.idx = idx; a.W = W; a.mean = rmean; a.rstd = rvar; a.stat_is_var = 1;
    a.bias = unbinarize_bias; a.gamma = gamma; a.beta = beta;
    a.O = node_size; a.F = frame_size; a.xs = frame_stride; a.ys = frame_stride; a.lut_binarize = lut_binarize; a.binary = 1;
    return launch_forward<true, PH_NORM, true>(a, 2048, as_stream(stream));
}

static int dl6_backward_args(BwdArgs &a, const void *x, const float *dy, float *dx, const int *idx, const float *W, float *dW,
                             const float *mean, const float *rstd, float gamma, float beta, float bias, int I, int O, int F,
                             long long xs, long long fs, int lut_binarize, int binary)
{
    int rc = check_common(x, dx, idx, W, O, F, fs);
    if (rc) return rc;
    BB200_REQUIRE_PTR(dy); BB200_REQUIRE_PTR(dW); BB200_REQUIRE_PTR(mean); BB200_REQUIRE_PTR(rstd);
    BB200_REQUIRE(I >= 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE(fs >= F, BBCU_ERR_BAD_STRIDE);
    a = BwdArgs{};
    a.x = x; a.dy = dy; a.dx = dx; a.idx = idx; a.W = W; a.dW = dW; a.mean = mean; a.rstd = rstd;
    a.gamma = gamma; a.beta = beta; a.bias = bias;
    a.O = O; a.F = F; a.xs = xs; a.dys = fs; a.dxs = fs; a.lut_binarize = lut_binarize; a.binary = binary;
    return BBCU_OK;
}

extern "C" int bbcu_fp32_DifferentiableLut6_Backward(const float *x, const float *dy, float *dx, float *dx_tmp, const int *idx, const int *rev,
                                                     const float *W, float *dW, const float *mean, const float *rstd, float *dmean_tmp,
                                                     float *dvar_tmp, float gamma, float beta, float unbinarize_bias, int reverse_index_stride,
                                                     int input_node_size, int output_node_size, int frame_size, int frame_stride,
                                                     int tmp_frame_size, int tmp_frame_stride, int lut_binarize, int binary_mode,
                                                     bbcu_stream_t stream)
{
    (void)rev; (void)reverse_index_stride; (void)tmp_frame_size;
    BB200_REQUIRE_PTR(dmean_tmp); BB200_REQUIRE_PTR(dvar_tmp);
    BwdArgs a;
    int rc = dl6_backward_args(a, x, dy, dx, idx, W, dW, mean, rstd, gamma, beta, unbinarize_bias, input_node_size, output_node_size, frame_size,
                               frame_stride, frame_stride, lut_binarize, binary_mode);
    if (rc) return rc;
    return backward_common<false>(a, true, frame_size > 0 ? frame_size : 1, dmean_tmp, dvar_tmp, nullptr, input_node_size, as_stream(stream),
                                  dx_tmp, dx_tmp_bytes(dx_tmp, output_node_size, tmp_frame_stride));
}

extern "C" int bbcu_bit_fp32_DifferentiableLut6_Backward(const int *x, const float *dy, float *dx, float *dx_tmp, const int *idx, const int *rev,
                                                         const float *W, float *dW, const float *mean, const float *rstd, float *dmean_tmp,
                                                         float *dvar_tmp, float gamma, float beta, float unbinarize_bias,
                                                         int reverse_index_stride, int input_node_size, int output_node_size, int frame_size,
                                                         int frame_stride, int x_frame_stride, int tmp_frame_size, int tmp_frame_stride,
                                                         int lut_binarize, bbcu_stream_t stream)
{
    (void)dx_tmp; (void)rev; (void)reverse_index_stride; (void)tmp_frame_size; (void)tmp_frame_stride;
    BB200_REQUIRE_PTR(dmean_tmp); BB200_REQUIRE_PTR(dvar_tmp);
    BB200_REQUIRE((long long)x_frame_stride * 32 >= frame_size, BBCU_ERR_BAD_STRIDE);
    BwdArgs a;
    int rc = dl6_backward_args(a, x, dy, dx, idx, W, dW, mean, rstd, gamma, beta, unbinarize_bias, input_node_size, output_node_size, frame_size,
                               x_frame_stride, frame_stride, lut_binarize, 1);
    if (rc) return rc;
    return backward_common<true>(a, true, frame_size > 0 ? frame_size : 1, dmean_tmp, dvar_tmp, nullptr, input_node_size, as_stream(stream));
}

extern "C" int bbcu_fp32_DifferentiableLut6_BackwardStats(const float *x, const float *dy, const int *idx, const float *W, const float *mean,
                                                          const float *rstd, double *dev_sums, float gamma, float beta, float unbinarize_bias,
                                                          int node_size, int frame_size, int frame_stride, int lut_binarize, int binary_mode,
                                                          bbcu_stream_t stream)
{
    int rc = check_common(x, dev_sums, idx, W, node_size, frame_size, frame_stride);
    if (rc) return rc;
    BB200_REQUIRE_PTR(dy); BB200_REQUIRE_PTR(mean); BB200_REQUIRE_PTR(rstd);
    BB200_REQUIRE(frame_stride >= frame_size, BBCU_ERR_BAD_STRIDE);
    cudaStream_t st = as_stream(stream);
    if (binary_mode) {        // two-valued inputs: the sums follow from the per-pattern dy sums (binary_mode.cu)
        rc = bit_backward_stats_by_table(true, x, dy, idx, W, mean, rstd, dev_sums, gamma, beta, unbinarize_bias, node_size, frame_size, frame_stride,
                                         frame_stride, lut_binarize, st);
        if (rc != BBCU_ERR_NO_MEMORY) return rc;
    }
    BB200_CUDA(cudaMemsetAsync(dev_sums, 0, sizeof(double) * 2 * (size_t)node_size, st));
    if (node_size == 0 || frame_size == 0) return BBCU_OK;
    BwdArgs a = {};
    a.x = x; a.dy = dy; a.idx = idx; a.W = W; a.mean = mean; a.rstd = rstd; a.sums = dev_sums;
    a.gamma = gamma; a.beta = beta; a.bias = unbinarize_bias;
    a.O = node_size; a.F = frame_size; a.xs = frame_stride; a.dys = frame_stride; a.lut_binarize = lut_binarize; a.binary = binary_mode;
    a.groups = (a.O + kWarpsPerCta - 1) / kWarpsPerCta;
    if (backward_stats_pipe(a, st, &rc)) return rc;
    a.T = frame_tile(3LL * a.O, 32, a.groups, a.F, 2048);
    const long long blocks = (long long)((a.F + a.T - 1) / a.T) * a.groups;
    BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
    k_lut6_backward_stats<false><<<(unsigned)blocks, kWarpsPerCta * 32, 0, st>>>(a);
    return launch_status();
}

extern "C" int bbcu_fp32_DifferentiableLut6_BackwardStatsFromOutput(const float *y, const float *dy, const float *rstd, double *dev_sums,
                                                                    float gamma, float beta, int node_size, int frame_size,
                                                                    int frame_stride, int binary_mode, bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(y); BB200_REQUIRE_PTR(dy); BB200_REQUIRE_PTR(rstd); BB200_REQUIRE_PTR(dev_sums);
    BB200_REQUIRE(node_size >= 0 && frame_size >= 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE(binary_mode == 0, BBCU_ERR_BAD_SIZE);          // a binarised output does not carry the pre-activation value
    BB200_REQUIRE(frame_stride >= frame_size, BBCU_ERR_BAD_STRIDE);
    cudaStream_t st = as_stream(stream);
    BB200_CUDA(cudaMemsetAsync(dev_sums, 0, sizeof(double) * 2 * (size_t)node_size, st));
    if (node_size == 0 || frame_size == 0) return BBCU_OK;
    const int chunks = (frame_size + 8191) / 8192;
    BB200_REQUIRE((long long)node_size * chunks < (1LL << 31), BBCU_ERR_TOO_LARGE);
    k_dl6_backward_stats_from_y<<<node_size * chunks, 256, 0, st>>>(y, dy, rstd, dev_sums, gamma, beta, frame_size, frame_stride, frame_stride,
                                                                    chunks);
    return launch_status();
}

extern "C" int bbcu_fp32_DifferentiableLut6_BackwardApply(const float *x, const float *dy, float *dx, const int *idx, const float *W, float *dW,
                                                          const float *mean, const float *rstd, const double *dev_sums, float *dmean_tmp,
                                                          float *dvar_tmp, float gamma, float beta, float unbinarize_bias, int input_node_size,
                                                          int output_node_size, int frame_size, int frame_stride, long long total_frame_size,
                                                          int lut_binarize, int binary_mode, bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(dev_sums); BB200_REQUIRE_PTR(dmean_tmp); BB200_REQUIRE_PTR(dvar_tmp);
    BB200_REQUIRE(total_frame_size >= frame_size && total_frame_size > 0, BBCU_ERR_BAD_SIZE);
    BwdArgs a;
    int rc = dl6_backward_args(a, x, dy, dx, idx, W, dW, mean, rstd, gamma, beta, unbinarize_bias, input_node_size, output_node_size, frame_size,
                               frame_stride, frame_stride, lut_binarize, binary_mode);
    if (rc) return rc;
    return backward_common<false>(a, true, total_frame_size, dmean_tmp, dvar_tmp, dev_sums, input_node_size, as_stream(stream));
}
