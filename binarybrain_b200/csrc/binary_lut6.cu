// BinaryLut6: bit-packed 6-input LUT inference forward.
//
// Semantics of BinaryBrain include/bb/BinaryLutN.h:436-463: for every frame the six input bits form an
// index (input k -> bit k) into the node's 64-entry truth table.  Frames are processed 32 per word
// as a multiplexer tree over whole words: 32 two-way selects on x0 between table constants, then
// 16/8/4/2/1 selects on x1..x5 -- 63 three-input logic ops (LOP3) per 32 frames, against the 448 of
// the reference kernel's 64 masked AND chains (cuda/BinaryLut6.cu:82-160).
//
// Mapping: one warp per output node, one 128-bit load per lane and input row, so a warp reads 512
// contiguous bytes of each of its six rows per iteration; CTAs of consecutive node groups share a
// word tile so the tile's input rows stay in L2 for the ~6 nodes that read each of them.

#include "common.cuh"
#include "async_copy.cuh"

namespace bb200 {

constexpr int kBlWarps = 8;

struct BlArgs {
    const uint32_t *x;
    uint32_t *y;
    const int *idx;
    const int *table;
    int O, nwords, Tw, groups;
    long long stride;
};

// level-1 select masks of a node: v_k = (x0 & A[k]) ^ B[k] equals table bit 2k (x0 = 0) / 2k+1 (x0 = 1)
__device__ __forceinline__ uint32_t lut6_word(uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3, uint32_t x4, uint32_t x5,
                                              const uint32_t (&A)[32], const uint32_t (&B)[32])
{
    uint32_t v[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) v[k] = (x0 & A[k]) ^ B[k];
#pragma unroll
    for (int k = 0; k < 16; ++k) v[k] = (v[2 * k] & ~x1) | (v[2 * k + 1] & x1);
#pragma unroll
    for (int k = 0; k < 8; ++k)  v[k] = (v[2 * k] & ~x2) | (v[2 * k + 1] & x2);
#pragma unroll
    for (int k = 0; k < 4; ++k)  v[k] = (v[2 * k] & ~x3) | (v[2 * k + 1] & x3);
#pragma unroll
    for (int k = 0; k < 2; ++k)  v[k] = (v[2 * k] & ~x4) | (v[2 * k + 1] & x4);
    return (v[0] & ~x5) | (v[1] & x5);
}

// Word-at-a-time kernel for rows that are not 16-byte aligned (any stride, any base address).
__global__ void __launch_bounds__(kBlWarps * 32)
k_binary_lut6(const BlArgs a)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / a.groups;
    const int node = (blockIdx.x % a.groups) * kBlWarps + warp;
    if (node >= a.O) return;

    const uint32_t t0 = (uint32_t)__ldg(a.table + 2 * (size_t)node);
    const uint32_t t1 = (uint32_t)__ldg(a.table + 2 * (size_t)node + 1);
    uint32_t A[32], B[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) {
        const uint32_t t  = (k < 16) ? t0 : t1;
        const uint32_t lo = (t >> ((2 * k) & 31)) & 1u, hi = (t >> ((2 * k + 1) & 31)) & 1u;
        B[k] = 0u - lo;
        A[k] = 0u - (lo ^ hi);
    }
    const uint32_t *rows[6];
#pragma unroll
    for (int j = 0; j < 6; ++j) rows[j] = a.x + (size_t)__ldg(a.idx + (size_t)node * 6 + j) * a.stride;
    uint32_t *yrow = a.y + (size_t)node * a.stride;

    const int w_begin = tile * a.Tw;
    const int w_end   = min(a.nwords, w_begin + a.Tw);
    for (int w = w_begin + lane; w < w_end; w += 32) {
        uint32_t xv[6];
#pragma unroll
        for (int j = 0; j < 6; ++j) xv[j] = __ldg(rows[j] + w);
        yrow[w] = lut6_word(xv[0], xv[1], xv[2], xv[3], xv[4], xv[5], A, B);
    }
}

// ---------------------------------------------------------------------------------------------
// Two-pipe variant (the one the launcher uses for aligned rows).
//   * Level 1 of the tree only ever produces one of {0, x0, ~x0, ~0}.  In two's complement that is
//     x0 * a + b with (a, b) in {(0,0), (1,0), (-1,-1), (0,-1)}: an integer multiply-add, which issues to the
//     FMA pipe and leaves the 31 selects of levels 2..6 to the INT/logic pipe, so the two pipes split the
//     63 ops per 32 frames about evenly instead of the logic pipe taking all of them.
//   * The 32 (a, b) pairs of a node are derived by 32 lanes in parallel (lane k does pair k) and exchanged
//     through shared memory, instead of every lane deriving all 64 values.
//   * Each lane carries 8 words (two 128-bit loads per input row) per iteration.
// ---------------------------------------------------------------------------------------------
template <typename AB>     // AB: int2[32] in registers, or a pointer to the warp's 32 pairs in shared memory
__device__ __forceinline__ uint32_t lut6_word_imad(uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3, uint32_t x4, uint32_t x5,
                                                   const AB &ab)
{
    uint32_t v[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) v[k] = x0 * (uint32_t)ab[k].x + (uint32_t)ab[k].y;
#pragma unroll
    for (int k = 0; k < 16; ++k) v[k] = (v[2 * k] & ~x1) | (v[2 * k + 1] & x1);
#pragma unroll
    for (int k = 0; k < 8; ++k)  v[k] = (v[2 * k] & ~x2) | (v[2 * k + 1] & x2);
#pragma unroll
    for (int k = 0; k < 4; ++k)  v[k] = (v[2 * k] & ~x3) | (v[2 * k + 1] & x3);
#pragma unroll
    for (int k = 0; k < 2; ++k)  v[k] = (v[2 * k] & ~x4) | (v[2 * k + 1] & x4);
    return (v[0] & ~x5) | (v[1] & x5);
}

__global__ void __launch_bounds__(kBlWarps * 32)
k_binary_lut6_2pipe(const BlArgs a)
{
    __shared__ int2 s_ab[kBlWarps][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / a.groups;
    const int node = (blockIdx.x % a.groups) * kBlWarps + warp;
    if (node >= a.O) return;
    {
        // lane k: table bits 2k (x0 = 0) and 2k+1 (x0 = 1) -> (a, b)
        const uint32_t t  = (uint32_t)__ldg(a.table + 2 * (size_t)node + (lane >> 4));
        const uint32_t lo = (t >> ((2 * lane) & 31)) & 1u, hi = (t >> ((2 * lane + 1) & 31)) & 1u;
        s_ab[warp][lane] = make_int2((int)hi - (int)lo, -(int)lo);
        __syncwarp();
    }
    int2 ab[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) ab[k] = s_ab[warp][k];
    const uint32_t *rows[6];
#pragma unroll
    for (int j = 0; j < 6; ++j) rows[j] = a.x + (size_t)__ldg(a.idx + (size_t)node * 6 + j) * a.stride;
    uint32_t *yrow = a.y + (size_t)node * a.stride;

    const int w_begin = tile * a.Tw;
    const int w_end   = min(a.nwords, w_begin + a.Tw);
    for (int w = w_begin + 4 * lane; w < w_end; w += 256) {
        const bool second = (w + 128) < w_end;
        uint4 lo[6], hi[6];
#pragma unroll
        for (int j = 0; j < 6; ++j) {
            lo[j] = __ldg(reinterpret_cast<const uint4 *>(rows[j] + w));
            hi[j] = second ? __ldg(reinterpret_cast<const uint4 *>(rows[j] + w + 128)) : make_uint4(0, 0, 0, 0);
        }
        uint4 o;
        o.x = lut6_word_imad(lo[0].x, lo[1].x, lo[2].x, lo[3].x, lo[4].x, lo[5].x, ab);
        o.y = lut6_word_imad(lo[0].y, lo[1].y, lo[2].y, lo[3].y, lo[4].y, lo[5].y, ab);
        o.z = lut6_word_imad(lo[0].z, lo[1].z, lo[2].z, lo[3].z, lo[4].z, lo[5].z, ab);
        o.w = lut6_word_imad(lo[0].w, lo[1].w, lo[2].w, lo[3].w, lo[4].w, lo[5].w, ab);
        *reinterpret_cast<uint4 *>(yrow + w) = o;
        if (second) {
            o.x = lut6_word_imad(hi[0].x, hi[1].x, hi[2].x, hi[3].x, hi[4].x, hi[5].x, ab);
            o.y = lut6_word_imad(hi[0].y, hi[1].y, hi[2].y, hi[3].y, hi[4].y, hi[5].y, ab);
            o.z = lut6_word_imad(hi[0].z, hi[1].z, hi[2].z, hi[3].z, hi[4].z, hi[5].z, ab);
            o.w = lut6_word_imad(hi[0].w, hi[1].w, hi[2].w, hi[3].w, hi[4].w, hi[5].w, ab);
            *reinterpret_cast<uint4 *>(yrow + w + 128) = o;
        }
    }
}

// Depth-first multiplexer tree over NW words at once.  A level-1 node costs one 64-bit shared-memory read of its
// (a, b) pair, shared by all NW words; walking depth first keeps about one live value per level and word, so eight
// words fit in registers and the pair reads amortise to four per word instead of thirty-two.
template <int L, int K, int NW>
struct MuxTree {
    static __device__ __forceinline__ void eval(const int2 *ab, const uint32_t (&x)[6][NW], uint32_t (&out)[NW])
    {
        uint32_t lo[NW], hi[NW];
        MuxTree<L - 1, 2 * K, NW>::eval(ab, x, lo);
        MuxTree<L - 1, 2 * K + 1, NW>::eval(ab, x, hi);
#pragma unroll
        for (int w = 0; w < NW; ++w) out[w] = (lo[w] & ~x[L - 1][w]) | (hi[w] & x[L - 1][w]);
    }
};

template <int K, int NW>
struct MuxTree<1, K, NW> {
    static __device__ __forceinline__ void eval(const int2 *ab, const uint32_t (&x)[6][NW], uint32_t (&out)[NW])
    {
        const int2 p = ab[K];
#pragma unroll
        for (int w = 0; w < NW; ++w) out[w] = x[0][w] * (uint32_t)p.x + (uint32_t)p.y;
    }
};

// ---------------------------------------------------------------------------------------------
// Persistent, bulk-copy-pipelined variant (aligned rows; the launcher's default).
// Work item = (word tile of 256 words, group of 8 nodes); CTA c takes items c, c + gridDim, ... so the CTAs in
// flight sweep the node groups of one tile together and the tile's rows stay in L2.  Each warp owns one node of
// the group and runs its own two-stage pipeline: lane 0 starts six 1 KiB bulk copies (one per gathered row) for
// item j+2 as soon as item j has been read out of shared memory into registers, then the warp computes item j
// while the copies of j+1 and j+2 are in flight.  No warp ever waits on a load it has only just issued, and no
// CTA-wide barrier exists after set-up.
// ---------------------------------------------------------------------------------------------
constexpr int kPipeCtas   = 2;                        // resident CTAs per SM
constexpr int kPipeNW     = 8;                        // words per lane and item
constexpr int kPipeWords  = 32 * kPipeNW;             // words per row segment and item (1 KiB)
constexpr int kPipeStages = 2;
// dynamic shared memory layout: [rows: warp x stage x 6 x 256 words][barriers: warp x stage, padded to 128 B][level-1 pairs: warp x 32 x int2]
constexpr int kPipeRowsBytes = kBlWarps * kPipeStages * 6 * kPipeWords * 4;
constexpr int kPipeBarBytes  = 128;
constexpr int kPipeAbBytes   = kBlWarps * 32 * 8;
constexpr int kPipeSmem      = kPipeRowsBytes + kPipeBarBytes + kPipeAbBytes;
static_assert(kBlWarps * kPipeStages * 8 <= kPipeBarBytes, "barrier block too small");

// Position of a work item, advanced incrementally (item index + gridDim) so that no division runs per item.
struct PipePos {
    int tile, group;
};

__device__ __forceinline__ PipePos pipe_advance(PipePos p, int dt, int dg, int groups)
{
    p.group += dg;
    p.tile += dt;
    if (p.group >= groups) { p.group -= groups; ++p.tile; }
    return p;
}

// Lanes 0..5 each start the bulk copy of one gathered row segment (one instruction issue covers all six); lane 0 has
// armed the barrier with the byte count just before.
// `row` is the lane's input row of the item's node (pipe_row), fetched an item earlier so that the copy does not wait for it.
__device__ __forceinline__ void pipe_issue(const BlArgs &a, PipePos pos, int row, int lane, uint32_t *stage, uint64_t *bar)
{
    const int w0    = pos.tile * kPipeWords;
    const uint32_t bytes = (uint32_t)min(kPipeWords, a.nwords - w0) * 4u;
    if (lane == 0) mbar_arrive_expect_tx(bar, 6u * bytes);
    __syncwarp();
    if (lane < 6) bulk_copy_g2s(stage + lane * kPipeWords, a.x + (size_t)row * a.stride + w0, bytes, bar);
}

__device__ __forceinline__ int pipe_row(const BlArgs &a, PipePos pos, int warp, int lane)
{
    const int node = min(pos.group * kBlWarps + warp, a.O - 1);
    return lane < 6 ? __ldg(a.idx + (size_t)node * 6 + lane) : 0;
}

__global__ void __launch_bounds__(kBlWarps * 32, kPipeCtas)
k_binary_lut6_pipe(const BlArgs a, int n_tiles, int *fault)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    uint32_t *s_rows = reinterpret_cast<uint32_t *>(smem_raw);                                   // [warp][stage][6][256]
    uint64_t *s_bar  = reinterpret_cast<uint64_t *>(smem_raw + kPipeRowsBytes);                   // [warp][stage]
    int2     *s_ab   = reinterpret_cast<int2 *>(smem_raw + kPipeRowsBytes + kPipeBarBytes);      // [warp][32]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t *my_rows = s_rows + (size_t)warp * kPipeStages * 6 * kPipeWords;
    uint64_t *my_bar  = s_bar + warp * kPipeStages;
    int2     *my_ab   = s_ab + warp * 32;

    if (lane == 0) {
        for (int s = 0; s < kPipeStages; ++s) mbar_init(my_bar + s, 1);
        mbar_init_fence();
    }
    __syncwarp();

    // items blockIdx, blockIdx + gridDim, ...: position of the current item and of the next two
    const int step = (int)gridDim.x;
    const int dt = step / a.groups, dg = step - dt * a.groups;
    PipePos p0;
    p0.tile  = (int)blockIdx.x / a.groups;
    p0.group = (int)blockIdx.x - p0.tile * a.groups;
    PipePos p1 = pipe_advance(p0, dt, dg, a.groups);
    PipePos p2 = pipe_advance(p1, dt, dg, a.groups);

    if (p0.tile < n_tiles) pipe_issue(a, p0, pipe_row(a, p0, warp, lane), lane, my_rows, my_bar);
    if (p1.tile < n_tiles) pipe_issue(a, p1, pipe_row(a, p1, warp, lane), lane, my_rows + 6 * kPipeWords, my_bar + 1);
    int row2 = p2.tile < n_tiles ? pipe_row(a, p2, warp, lane) : 0;          // input rows of item k+2, one item ahead of their use
    uint32_t tword = 0;
    if (p0.tile < n_tiles) tword = (uint32_t)__ldg(a.table + 2 * (size_t)min(p0.group * kBlWarps + warp, a.O - 1) + (lane >> 4));

    for (int k = 0; p0.tile < n_tiles; ++k) {
        const int s = k & 1;
        const uint32_t parity = (uint32_t)(k >> 1) & 1u;
        uint32_t *stage = my_rows + s * 6 * kPipeWords;
        const int node = p0.group * kBlWarps + warp;
        const bool store = node < a.O;
        const int w0 = p0.tile * kPipeWords;
        const int nw = min(kPipeWords, a.nwords - w0);

        // this node's level-1 (a, b) pairs; the table word of the NEXT item is fetched now and used next round
        {
            const uint32_t lo = (tword >> ((2 * lane) & 31)) & 1u, hi = (tword >> ((2 * lane + 1) & 31)) & 1u;
            __syncwarp();
            my_ab[lane] = make_int2((int)hi - (int)lo, -(int)lo);
            __syncwarp();
        }
        const bool have_next = p1.tile < n_tiles;
        if (have_next) tword = (uint32_t)__ldg(a.table + 2 * (size_t)min(p1.group * kBlWarps + warp, a.O - 1) + (lane >> 4));

        if (!mbar_wait(my_bar + s, parity)) {          // bounded: record the fault, let the other stage's copies land, leave
            if (lane == 0) atomicCAS(fault, 0, kFaultBarrierTimeout);
            if (have_next) mbar_wait(my_bar + (s ^ 1), (uint32_t)((k + 1) >> 1) & 1u);
            return;
        }
        const int w = 4 * lane;
        uint32_t xw[6][kPipeNW], o[kPipeNW];
#pragma unroll
        for (int j = 0; j < 6; ++j) {
#pragma unroll
            for (int h = 0; h < kPipeNW / 4; ++h) {
                const uint4 v = *reinterpret_cast<const uint4 *>(stage + j * kPipeWords + w + 128 * h);
                xw[j][4 * h] = v.x; xw[j][4 * h + 1] = v.y; xw[j][4 * h + 2] = v.z; xw[j][4 * h + 3] = v.w;
            }
        }
        __syncwarp();                                   // every lane has read the stage out
        if (p2.tile < n_tiles) {
            proxy_fence_async();                        // reads above (generic proxy) before the refill (async proxy)
            pipe_issue(a, p2, row2, lane, stage, my_bar + s);
        }
        const PipePos p3 = pipe_advance(p2, dt, dg, a.groups);
        if (p3.tile < n_tiles) row2 = pipe_row(a, p3, warp, lane);
        MuxTree<6, 0, kPipeNW>::eval(my_ab, xw, o);
        uint32_t *yrow = a.y + (size_t)min(node, a.O - 1) * a.stride + w0;
#pragma unroll
        for (int h = 0; h < kPipeNW / 4; ++h)
            if (store && w + 128 * h < nw) *reinterpret_cast<uint4 *>(yrow + w + 128 * h) = make_uint4(o[4 * h], o[4 * h + 1], o[4 * h + 2], o[4 * h + 3]);

        p0 = p1; p1 = p2; p2 = p3;
    }
}

}   // namespace bb200

using namespace bb200;

extern "C" int bbcu_bit_BinaryLut6_Forward(const int *x, int *y, const int *idx, const int *table, int node_size, int frame_size,
                                           int frame_stride, bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(x); BB200_REQUIRE_PTR(y); BB200_REQUIRE_PTR(idx); BB200_REQUIRE_PTR(table);
    BB200_REQUIRE(node_size >= 0 && frame_size >= 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE((long long)frame_stride * 32 >= frame_size, BBCU_ERR_BAD_STRIDE);
    if (node_size == 0 || frame_size == 0) return BBCU_OK;

    BlArgs a;
    a.x = reinterpret_cast<const uint32_t *>(x); a.y = reinterpret_cast<uint32_t *>(y); a.idx = idx; a.table = table;
    a.O = node_size; a.stride = frame_stride;
    a.nwords = (frame_size + 31) / 32;
    a.groups = (node_size + kBlWarps - 1) / kBlWarps;
    // 128-bit path: rows start 16-byte aligned and whole uint4 groups fit inside the row stride
    const bool vec = (frame_stride % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((reinterpret_cast<uintptr_t>(y) & 15) == 0);
    if (vec) a.nwords = (a.nwords + 3) & ~3;
    // word tile: frame_tile() counts in frames; a word is 32 of them
    const int tf = frame_tile(2LL * node_size, 1, a.groups, a.nwords * 32, 1024 * 32);
    a.Tw = ((tf / 32 + 127) / 128) * 128;
    const long long blocks = (long long)((a.nwords + a.Tw - 1) / a.Tw) * a.groups;
    BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
    if (vec) {
        // persistent pipeline: two CTAs per SM, each walking (tile, node group) items
        static bool attr_done[64] = {};              // the opt-in to > 48 KB of dynamic shared memory is per device
        const int dev_id = bbcu_GetDevice();
        bool attr_ok = dev_id >= 0 && dev_id < 64 && attr_done[dev_id];
        if (!attr_ok && dev_id >= 0 && dev_id < 64) {
            attr_ok = cudaFuncSetAttribute(k_binary_lut6_pipe, cudaFuncAttributeMaxDynamicSharedMemorySize, kPipeSmem) == cudaSuccess;
            attr_done[dev_id] = attr_ok;
            if (!attr_ok) cudaGetLastError();
        }
        int *fault = fault_word();
        if (attr_ok && fault != nullptr) {
            const long long n_items = (long long)((a.nwords + kPipeWords - 1) / kPipeWords) * a.groups;
            BB200_REQUIRE(n_items < (1LL << 31) - 4096, BBCU_ERR_TOO_LARGE);      // 32-bit item arithmetic in the kernel
            long long grid = (long long)kPipeCtas * device_info().sm_count;
            if (grid > n_items) grid = n_items;
            k_binary_lut6_pipe<<<(unsigned)grid, kBlWarps * 32, kPipeSmem, as_stream(stream)>>>(a, (a.nwords + kPipeWords - 1) / kPipeWords, fault);
            return launch_status();
        }
    }
    // aligned rows without the shared-memory opt-in (or without a fault word): the non-pipelined 128-bit kernel; otherwise word loads
    if (vec) k_binary_lut6_2pipe<<<(unsigned)blocks, kBlWarps * 32, 0, as_stream(stream)>>>(a);
    else     k_binary_lut6<<<(unsigned)blocks, kBlWarps * 32, 0, as_stream(stream)>>>(a);
    return launch_status();
}

extern "C" int bbcu_bit_BinatyLut6_Forward(const int *x, int *y, const int *idx, const int *table, int node_size, int frame_size,
                                           int frame_stride, bbcu_stream_t stream)
{
    return bbcu_bit_BinaryLut6_Forward(x, y, idx, table, node_size, frame_size, frame_stride, stream);
}
