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

// ---------------------------------------------------------------------------------------------
// Truth-table-immediate variant (aligned rows).
// lop3.b32 evaluates ANY three-input boolean function in one instruction, the function being an 8-bit immediate.  Byte b of a
// node's 64-bit table is exactly the function of (x0, x1, x2) that applies where x3 + 2 x4 + 4 x5 = b, so a word costs eight lop3
// with the table bytes as immediates and seven selects on x3, x4, x5: 15 logic operations instead of 63.  The immediates are
// instruction text, so each table byte is dispatched through one indexed branch (brx.idx) into 256 case bodies that hold the
// lop3 for all 16 words of a lane; the byte is warp-uniform (one node per warp), so the branch never diverges and its cost --
// the branch and the instruction fetch of a cold case body -- is spread over 16 words.  The eight partial results are folded as
// a binary counter does (s0 waits for its odd neighbour, s1 for the next pair, s2 for the upper half).  The whole per-item
// evaluation is one asm statement: branch targets must be labels of the block that holds the table, and mutable PTX registers
// keep the partial results in place across the eight trips.
// Operands: %0-%15 y, %16-%31 x0, %32-%47 x1, %48-%63 x2, %64-%79 x3, %80-%95 x4, %96-%111 x5, %112 / %113 the table words.
// Staging: every lane copies, with cp.async, the 16-byte pieces of the six rows that it will itself read, two items ahead
// (two-stage ring per warp): no barrier and no cross-lane dependence.
// ---------------------------------------------------------------------------------------------
constexpr int kImmNW     = 16;                         // words per lane and item (four 128-bit pieces per row)
constexpr int kImmWords  = 32 * kImmNW;                // words per row segment and item
constexpr int kImmStages = 2;
constexpr int kImmStageBytes = 6 * kImmWords * 4;
constexpr int kImmSmem   = kBlWarps * kImmStages * kImmStageBytes;
static_assert(kImmSmem <= 227 * 1024, "one CTA per SM must fit");

#define BB200_LOPS(imm) \
    "lop3.b32 p0, %48, %32, %16, " imm ";\n\t" "lop3.b32 p1, %49, %33, %17, " imm ";\n\t" "lop3.b32 p2, %50, %34, %18, " imm ";\n\t" "lop3.b32 p3, %51, %35, %19, " imm ";\n\t" \
    "lop3.b32 p4, %52, %36, %20, " imm ";\n\t" "lop3.b32 p5, %53, %37, %21, " imm ";\n\t" "lop3.b32 p6, %54, %38, %22, " imm ";\n\t" "lop3.b32 p7, %55, %39, %23, " imm ";\n\t" \
    "lop3.b32 p8, %56, %40, %24, " imm ";\n\t" "lop3.b32 p9, %57, %41, %25, " imm ";\n\t" "lop3.b32 p10, %58, %42, %26, " imm ";\n\t" "lop3.b32 p11, %59, %43, %27, " imm ";\n\t" \
    "lop3.b32 p12, %60, %44, %28, " imm ";\n\t" "lop3.b32 p13, %61, %45, %29, " imm ";\n\t" "lop3.b32 p14, %62, %46, %30, " imm ";\n\t" "lop3.b32 p15, %63, %47, %31, " imm ";\n\t"
#define BB200_CASE(h, l) "T" #h #l ":\n\t" BB200_LOPS("0x" #h #l) "bra.uni TEND;\n\t"
#define BB200_ROW(h)                                                                                                                        \
    BB200_CASE(h, 0) BB200_CASE(h, 1) BB200_CASE(h, 2) BB200_CASE(h, 3) BB200_CASE(h, 4) BB200_CASE(h, 5) BB200_CASE(h, 6) BB200_CASE(h, 7) \
    BB200_CASE(h, 8) BB200_CASE(h, 9) BB200_CASE(h, A) BB200_CASE(h, B) BB200_CASE(h, C) BB200_CASE(h, D) BB200_CASE(h, E) BB200_CASE(h, F)
#define BB200_TGT(h)                                                                                                                        \
    "T" #h "0, T" #h "1, T" #h "2, T" #h "3, T" #h "4, T" #h "5, T" #h "6, T" #h "7, T" #h "8, T" #h "9, T" #h "A, T" #h "B, T" #h "C, T" #h "D, T" #h "E, T" #h "F"

// y[w] = table[x0[w] + 2 x1[w] + 4 x2[w] + 8 x3[w] + 16 x4[w] + 32 x5[w]] bitwise, for the 16 words of a lane
__device__ __forceinline__ void lut6_words_by_immediates(uint32_t (&y)[16], const uint32_t (&x)[6][16], uint32_t table_lo, uint32_t table_hi)
{
    asm volatile(
        "{\n\t"
        ".reg .u32 p<16>, s0_<16>, s1_<16>, s2_<16>, t<16>;\n\t"
        ".reg .u32 b, byte, sh, tw, c;\n\t"
        ".reg .pred q;\n\t"
        "mov.u32 b, 0;\n\t"
        "LOOP:\n\t"
        "setp.lt.u32 q, b, 4;\n\t"
        "selp.u32 tw, %112, %113, q;\n\t"
        "and.b32 sh, b, 3;\n\t"
        "shl.b32 sh, sh, 3;\n\t"
        "shr.u32 byte, tw, sh;\n\t"
        "and.b32 byte, byte, 255;\n\t"
        "TBL: .branchtargets " BB200_TGT(0) ", " BB200_TGT(1) ", " BB200_TGT(2) ", " BB200_TGT(3) ", " BB200_TGT(4) ", " BB200_TGT(5) ", "
        BB200_TGT(6) ", " BB200_TGT(7) ", " BB200_TGT(8) ", " BB200_TGT(9) ", " BB200_TGT(A) ", " BB200_TGT(B) ", " BB200_TGT(C) ", "
        BB200_TGT(D) ", " BB200_TGT(E) ", " BB200_TGT(F) ";\n\t"
        "brx.idx byte, TBL;\n\t"
        BB200_ROW(0) BB200_ROW(1) BB200_ROW(2) BB200_ROW(3) BB200_ROW(4) BB200_ROW(5) BB200_ROW(6) BB200_ROW(7)
        BB200_ROW(8) BB200_ROW(9) BB200_ROW(A) BB200_ROW(B) BB200_ROW(C) BB200_ROW(D) BB200_ROW(E) BB200_ROW(F)
        "TEND:\n\t"
        "and.b32 c, b, 1;\n\t"
        "setp.ne.u32 q, c, 0;\n\t"
        "@q bra.uni ODD;\n\t"
        "mov.u32 s0_0, p0;\n\tmov.u32 s0_1, p1;\n\tmov.u32 s0_2, p2;\n\tmov.u32 s0_3, p3;\n\tmov.u32 s0_4, p4;\n\tmov.u32 s0_5, p5;\n\tmov.u32 s0_6, p6;\n\tmov.u32 s0_7, p7;\n\tmov.u32 s0_8, p8;\n\tmov.u32 s0_9, p9;\n\tmov.u32 s0_10, p10;\n\tmov.u32 s0_11, p11;\n\tmov.u32 s0_12, p12;\n\tmov.u32 s0_13, p13;\n\tmov.u32 s0_14, p14;\n\tmov.u32 s0_15, p15;\n\t"
        "bra.uni NEXT;\n\t"
        "ODD:\n\t"
        "lop3.b32 t0, %64, p0, s0_0, 0xCA;\n\tlop3.b32 t1, %65, p1, s0_1, 0xCA;\n\tlop3.b32 t2, %66, p2, s0_2, 0xCA;\n\tlop3.b32 t3, %67, p3, s0_3, 0xCA;\n\tlop3.b32 t4, %68, p4, s0_4, 0xCA;\n\tlop3.b32 t5, %69, p5, s0_5, 0xCA;\n\tlop3.b32 t6, %70, p6, s0_6, 0xCA;\n\tlop3.b32 t7, %71, p7, s0_7, 0xCA;\n\tlop3.b32 t8, %72, p8, s0_8, 0xCA;\n\tlop3.b32 t9, %73, p9, s0_9, 0xCA;\n\tlop3.b32 t10, %74, p10, s0_10, 0xCA;\n\tlop3.b32 t11, %75, p11, s0_11, 0xCA;\n\tlop3.b32 t12, %76, p12, s0_12, 0xCA;\n\tlop3.b32 t13, %77, p13, s0_13, 0xCA;\n\tlop3.b32 t14, %78, p14, s0_14, 0xCA;\n\tlop3.b32 t15, %79, p15, s0_15, 0xCA;\n\t"
        "and.b32 c, b, 2;\n\t"
        "setp.ne.u32 q, c, 0;\n\t"
        "@q bra.uni PAIR;\n\t"
        "mov.u32 s1_0, t0;\n\tmov.u32 s1_1, t1;\n\tmov.u32 s1_2, t2;\n\tmov.u32 s1_3, t3;\n\tmov.u32 s1_4, t4;\n\tmov.u32 s1_5, t5;\n\tmov.u32 s1_6, t6;\n\tmov.u32 s1_7, t7;\n\tmov.u32 s1_8, t8;\n\tmov.u32 s1_9, t9;\n\tmov.u32 s1_10, t10;\n\tmov.u32 s1_11, t11;\n\tmov.u32 s1_12, t12;\n\tmov.u32 s1_13, t13;\n\tmov.u32 s1_14, t14;\n\tmov.u32 s1_15, t15;\n\t"
        "bra.uni NEXT;\n\t"
        "PAIR:\n\t"
        "lop3.b32 t0, %80, t0, s1_0, 0xCA;\n\tlop3.b32 t1, %81, t1, s1_1, 0xCA;\n\tlop3.b32 t2, %82, t2, s1_2, 0xCA;\n\tlop3.b32 t3, %83, t3, s1_3, 0xCA;\n\tlop3.b32 t4, %84, t4, s1_4, 0xCA;\n\tlop3.b32 t5, %85, t5, s1_5, 0xCA;\n\tlop3.b32 t6, %86, t6, s1_6, 0xCA;\n\tlop3.b32 t7, %87, t7, s1_7, 0xCA;\n\tlop3.b32 t8, %88, t8, s1_8, 0xCA;\n\tlop3.b32 t9, %89, t9, s1_9, 0xCA;\n\tlop3.b32 t10, %90, t10, s1_10, 0xCA;\n\tlop3.b32 t11, %91, t11, s1_11, 0xCA;\n\tlop3.b32 t12, %92, t12, s1_12, 0xCA;\n\tlop3.b32 t13, %93, t13, s1_13, 0xCA;\n\tlop3.b32 t14, %94, t14, s1_14, 0xCA;\n\tlop3.b32 t15, %95, t15, s1_15, 0xCA;\n\t"
        "and.b32 c, b, 4;\n\t"
        "setp.ne.u32 q, c, 0;\n\t"
        "@q bra.uni TOP;\n\t"
        "mov.u32 s2_0, t0;\n\tmov.u32 s2_1, t1;\n\tmov.u32 s2_2, t2;\n\tmov.u32 s2_3, t3;\n\tmov.u32 s2_4, t4;\n\tmov.u32 s2_5, t5;\n\tmov.u32 s2_6, t6;\n\tmov.u32 s2_7, t7;\n\tmov.u32 s2_8, t8;\n\tmov.u32 s2_9, t9;\n\tmov.u32 s2_10, t10;\n\tmov.u32 s2_11, t11;\n\tmov.u32 s2_12, t12;\n\tmov.u32 s2_13, t13;\n\tmov.u32 s2_14, t14;\n\tmov.u32 s2_15, t15;\n\t"
        "bra.uni NEXT;\n\t"
        "TOP:\n\t"
        "lop3.b32 %0, %96, t0, s2_0, 0xCA;\n\tlop3.b32 %1, %97, t1, s2_1, 0xCA;\n\tlop3.b32 %2, %98, t2, s2_2, 0xCA;\n\tlop3.b32 %3, %99, t3, s2_3, 0xCA;\n\tlop3.b32 %4, %100, t4, s2_4, 0xCA;\n\tlop3.b32 %5, %101, t5, s2_5, 0xCA;\n\tlop3.b32 %6, %102, t6, s2_6, 0xCA;\n\tlop3.b32 %7, %103, t7, s2_7, 0xCA;\n\tlop3.b32 %8, %104, t8, s2_8, 0xCA;\n\tlop3.b32 %9, %105, t9, s2_9, 0xCA;\n\tlop3.b32 %10, %106, t10, s2_10, 0xCA;\n\tlop3.b32 %11, %107, t11, s2_11, 0xCA;\n\tlop3.b32 %12, %108, t12, s2_12, 0xCA;\n\tlop3.b32 %13, %109, t13, s2_13, 0xCA;\n\tlop3.b32 %14, %110, t14, s2_14, 0xCA;\n\tlop3.b32 %15, %111, t15, s2_15, 0xCA;\n\t"
        "NEXT:\n\t"
        "add.u32 b, b, 1;\n\t"
        "setp.lt.u32 q, b, 8;\n\t"
        "@q bra.uni LOOP;\n\t"
        "}"
        : "=&r"(y[0]), "=&r"(y[1]), "=&r"(y[2]), "=&r"(y[3]), "=&r"(y[4]), "=&r"(y[5]), "=&r"(y[6]), "=&r"(y[7]), "=&r"(y[8]), "=&r"(y[9]), "=&r"(y[10]), "=&r"(y[11]), "=&r"(y[12]), "=&r"(y[13]), "=&r"(y[14]), "=&r"(y[15])
        : "r"(x[0][0]), "r"(x[0][1]), "r"(x[0][2]), "r"(x[0][3]), "r"(x[0][4]), "r"(x[0][5]), "r"(x[0][6]), "r"(x[0][7]), "r"(x[0][8]), "r"(x[0][9]), "r"(x[0][10]), "r"(x[0][11]), "r"(x[0][12]), "r"(x[0][13]), "r"(x[0][14]), "r"(x[0][15]), "r"(x[1][0]), "r"(x[1][1]), "r"(x[1][2]), "r"(x[1][3]), "r"(x[1][4]), "r"(x[1][5]), "r"(x[1][6]), "r"(x[1][7]), "r"(x[1][8]), "r"(x[1][9]), "r"(x[1][10]), "r"(x[1][11]), "r"(x[1][12]), "r"(x[1][13]), "r"(x[1][14]), "r"(x[1][15]), "r"(x[2][0]), "r"(x[2][1]), "r"(x[2][2]), "r"(x[2][3]), "r"(x[2][4]), "r"(x[2][5]), "r"(x[2][6]), "r"(x[2][7]), "r"(x[2][8]), "r"(x[2][9]), "r"(x[2][10]), "r"(x[2][11]), "r"(x[2][12]), "r"(x[2][13]), "r"(x[2][14]), "r"(x[2][15]), "r"(x[3][0]), "r"(x[3][1]), "r"(x[3][2]), "r"(x[3][3]), "r"(x[3][4]), "r"(x[3][5]), "r"(x[3][6]), "r"(x[3][7]), "r"(x[3][8]), "r"(x[3][9]), "r"(x[3][10]), "r"(x[3][11]), "r"(x[3][12]), "r"(x[3][13]), "r"(x[3][14]), "r"(x[3][15]), "r"(x[4][0]), "r"(x[4][1]), "r"(x[4][2]), "r"(x[4][3]), "r"(x[4][4]), "r"(x[4][5]), "r"(x[4][6]), "r"(x[4][7]), "r"(x[4][8]), "r"(x[4][9]), "r"(x[4][10]), "r"(x[4][11]), "r"(x[4][12]), "r"(x[4][13]), "r"(x[4][14]), "r"(x[4][15]), "r"(x[5][0]), "r"(x[5][1]), "r"(x[5][2]), "r"(x[5][3]), "r"(x[5][4]), "r"(x[5][5]), "r"(x[5][6]), "r"(x[5][7]), "r"(x[5][8]), "r"(x[5][9]), "r"(x[5][10]), "r"(x[5][11]), "r"(x[5][12]), "r"(x[5][13]), "r"(x[5][14]), "r"(x[5][15]), "r"(table_lo), "r"(table_hi));
}
#undef BB200_LOPS
#undef BB200_CASE
#undef BB200_ROW
#undef BB200_TGT

__global__ void __launch_bounds__(kBlWarps * 32, 1)
k_binary_lut6_imm(const BlArgs a, int n_tiles)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t *my = reinterpret_cast<uint32_t *>(smem_raw) + (size_t)warp * kImmStages * 6 * kImmWords;

    const int step = (int)gridDim.x;
    const int dt = step / a.groups, dg = step - dt * a.groups;
    PipePos pi;                                        // copy side: two items ahead
    pi.tile  = (int)blockIdx.x / a.groups;
    pi.group = (int)blockIdx.x - pi.tile * a.groups;
    PipePos pc = pi;                                   // arithmetic side
    int row_i = pi.tile < n_tiles ? pipe_row(a, pi, warp, lane) : 0;
    int row_n;
    {
        const PipePos t = pipe_advance(pi, dt, dg, a.groups);
        row_n = t.tile < n_tiles ? pipe_row(a, t, warp, lane) : 0;
    }
    int ist = 0;
    auto issue = [&]() {
        if (pi.tile < n_tiles) {
            const int w0 = pi.tile * kImmWords + 4 * lane;
            uint32_t *st = my + ist * 6 * kImmWords + 4 * lane;
#pragma unroll
            for (int j = 0; j < 6; ++j) {
                const uint32_t *src = a.x + (size_t)__shfl_sync(0xffffffffu, row_i, j) * a.stride + w0;
#pragma unroll
                for (int h = 0; h < kImmNW / 4; ++h) {
                    const bool in_row = w0 + 128 * h < a.nwords;
                    cp_async16(st + j * kImmWords + 128 * h, in_row ? src + 128 * h : a.x, in_row);
                }
            }
            pi = pipe_advance(pi, dt, dg, a.groups);
            row_i = row_n;
            const PipePos t = pipe_advance(pi, dt, dg, a.groups);
            row_n = t.tile < n_tiles ? pipe_row(a, t, warp, lane) : 0;
        }
        cp_async_commit();
        ist ^= 1;
    };
    issue();
    issue();

    uint2 tab_n = make_uint2(0u, 0u);                   // the node's 64-bit table, one item ahead of its use
    if (pc.tile < n_tiles) tab_n = __ldg(reinterpret_cast<const uint2 *>(a.table) + min(pc.group * kBlWarps + warp, a.O - 1));
    int cst = 0;
    while (pc.tile < n_tiles) {
        const int node = pc.group * kBlWarps + warp;
        const bool store = node < a.O;
        const int w0 = pc.tile * kImmWords;
        const uint2 tab = tab_n;
        const PipePos pn = pipe_advance(pc, dt, dg, a.groups);
        if (pn.tile < n_tiles) tab_n = __ldg(reinterpret_cast<const uint2 *>(a.table) + min(pn.group * kBlWarps + warp, a.O - 1));

        cp_async_wait<1>();                             // the copies of this item (this lane's own pieces) have landed
        const uint32_t *st = my + cst * 6 * kImmWords + 4 * lane;
        cst ^= 1;
        uint32_t x[6][kImmNW], y[kImmNW];
#pragma unroll
        for (int j = 0; j < 6; ++j) {
#pragma unroll
            for (int h = 0; h < kImmNW / 4; ++h) {
                const uint4 v = *reinterpret_cast<const uint4 *>(st + j * kImmWords + 128 * h);
                x[j][4 * h] = v.x; x[j][4 * h + 1] = v.y; x[j][4 * h + 2] = v.z; x[j][4 * h + 3] = v.w;
            }
        }
        issue();                                        // refills the stage just read (each lane overwrites only what it has read itself)
        lut6_words_by_immediates(y, x, tab.x, tab.y);
        uint32_t *yrow = a.y + (size_t)min(node, a.O - 1) * a.stride + w0 + 4 * lane;
#pragma unroll
        for (int h = 0; h < kImmNW / 4; ++h)
            if (store && w0 + 4 * lane + 128 * h < a.nwords) *reinterpret_cast<uint4 *>(yrow + 128 * h) = make_uint4(y[4 * h], y[4 * h + 1], y[4 * h + 2], y[4 * h + 3]);
        pc = pn;
    }
    cp_async_wait<0>();
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

// The same operator through the truth-table-immediate kernel (k_binary_lut6_imm).  Kept as an entry point of its own because it is the
// formulation with the fewest logic operations (15 per word against 63) and nevertheless the slower one on B200 -- its case
// bodies are fetched cold from the instruction cache on every dispatch -- so that the comparison stays measurable.  Rows must be
// 16-byte aligned (stride a multiple of 4 words, aligned base pointers).
extern "C" int bbcu_bit_BinaryLut6_Forward_Lop3Immediate(const int *x, int *y, const int *idx, const int *table, int node_size, int frame_size,
                                                         int frame_stride, bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(x); BB200_REQUIRE_PTR(y); BB200_REQUIRE_PTR(idx); BB200_REQUIRE_PTR(table);
    BB200_REQUIRE(node_size >= 0 && frame_size >= 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE((long long)frame_stride * 32 >= frame_size, BBCU_ERR_BAD_STRIDE);
    BB200_REQUIRE(frame_stride % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(table) & 7) == 0, BBCU_ERR_BAD_STRIDE);
    if (node_size == 0 || frame_size == 0) return BBCU_OK;
    BlArgs a;
    a.x = reinterpret_cast<const uint32_t *>(x); a.y = reinterpret_cast<uint32_t *>(y); a.idx = idx; a.table = table;
    a.O = node_size; a.stride = frame_stride;
    a.nwords = ((frame_size + 31) / 32 + 3) & ~3;
    a.groups = (node_size + kBlWarps - 1) / kBlWarps;
    a.Tw = kImmWords;
    BB200_CUDA(cudaFuncSetAttribute(k_binary_lut6_imm, cudaFuncAttributeMaxDynamicSharedMemorySize, kImmSmem));
    const int n_tiles = (a.nwords + kImmWords - 1) / kImmWords;
    const long long n_items = (long long)n_tiles * a.groups;
    BB200_REQUIRE(n_items < (1LL << 31) - 4096, BBCU_ERR_TOO_LARGE);
    long long grid = device_info().sm_count;
    if (grid > n_items) grid = n_items;
    k_binary_lut6_imm<<<(unsigned)grid, kBlWarps * 32, kImmSmem, as_stream(stream)>>>(a, n_tiles);
    return launch_status();
}

extern "C" int bbcu_bit_BinatyLut6_Forward(const int *x, int *y, const int *idx, const int *table, int node_size, int frame_size,
                                           int frame_stride, bbcu_stream_t stream)
{
    return bbcu_bit_BinaryLut6_Forward(x, y, idx, table, node_size, frame_size, frame_stride, stream);
}
