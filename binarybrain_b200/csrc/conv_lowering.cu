// Convolution lowering around the per-pixel LUT layers of a LUT-CNN: Im2Col, Col2Im and MaxPooling.
//
// FrameBuffers are node-major and frame-contiguous, and lowering multiplies the frame axis by the output pixels:
// output frame  fo = fi * P + p  (fi = input frame, p = oy * OW + ox, P = OH * OW).  Every operator here is pure
// data movement, so the only thing to get right is that both the reads and the writes are made of full lines:
//   * Im2Col / Col2Im exchange the roles of "pixel" and "frame" (pixels are nodes on one side and part of the frame
//     index on the other), i.e. they are transposes through shared memory (fp32: a band of image rows x 32 frames per
//     block for Im2Col, 32 x 32 tiles for Col2Im and for images too wide for a band) or 32 x 32 bit-matrix transposes by
//     warp ballot (bit frames);
//   * MaxPooling keeps the frame axis and is a straight per-frame window scan.
//
// Semantics follow the reference's CPU branches:
//   Im2Col      include/bb/ConvolutionIm2Col.h:361-396 (forward, border modes :253-288), :439-482 (backward: only
//               positions inside the image receive gradient; replicated / reflected border copies send none back)
//   Col2Im      include/bb/ConvolutionCol2Im.h:205-221 (forward), :283-299 (backward)
//   MaxPooling  include/bb/MaxPooling.h:286-322 (fp32 forward: first maximum wins, argmax counts in-range window
//               positions), :369-394 (bit forward: OR), :600-629 (backward by argmax), :681-708 (bit layer backward:
//               the first set input bit takes the gradient)
#include "common.cuh"
#include "bit_transpose.cuh"

namespace bb200 {

namespace {

enum { kBorderConstant = 0, kBorderReflect = 1, kBorderReflect101 = 2, kBorderReplicate = 3, kBorderWrap = 4 };

struct Im2ColGeom {
    int x_stride, y_stride, x_offset, y_offset;
    int in_w, in_h, in_c, out_w, out_h, filter_w, filter_h, border_mode;
    int in_frames;
    long long in_fs, out_fs;          // frame strides in elements (floats / words)
};

__device__ __forceinline__ bool border_remap(int mode, int &x, int &y, int w, int h)
{
    switch (mode) {
    case kBorderReflect:
        if (x < 0) x = -x - 1;
        if (y < 0) y = -y - 1;
        if (x >= w) x = (w - 1) - (x - w);
        if (y >= h) y = (h - 1) - (y - h);
        return true;
    case kBorderReflect101:
        if (x < 0) x = -x;
        if (y < 0) y = -y;
        if (x >= w) x = (w - 2) - (x - w);
        if (y >= h) y = (h - 2) - (y - h);
        return true;
    case kBorderReplicate:
        if (x < 0) x = 0;
        if (y < 0) y = 0;
        if (x >= w) x = w - 1;
        if (y >= h) y = h - 1;
        return true;
    case kBorderWrap:
        if (x < 0) x += w;
        if (y < 0) y += h;
        if (x >= w) x -= w;
        if (y >= h) y -= h;
        return true;
    default:
        return false;
    }
}

// Input node read by output pixel p of output node (c, fy, fx), or -1 for the border value.
__device__ __forceinline__ int im2col_source(const Im2ColGeom &g, int c, int fy, int fx, int p)
{
    int iy = (p / g.out_w) * g.y_stride - g.y_offset + fy;
    int ix = (p % g.out_w) * g.x_stride - g.x_offset + fx;
    if (iy >= 0 && iy < g.in_h && ix >= 0 && ix < g.in_w) return (c * g.in_h + iy) * g.in_w + ix;
    if (border_remap(g.border_mode, ix, iy, g.in_w, g.in_h)) {
        // a remap that still misses the image (filter wider than the image) reads nothing
        if (iy >= 0 && iy < g.in_h && ix >= 0 && ix < g.in_w) return (c * g.in_h + iy) * g.in_w + ix;
    }
    return -1;
}

// --------------------------------------------------------------------------------------------- Im2Col fp32
// Block = one output node x 32 input frames x 128 output pixels (four 32 x 32 tiles, so that every thread has 16 independent
// loads in flight before the barrier).  Reads run along input frames, writes along pixels.
constexpr int kIm2ColTiles = 4;

__global__ void __launch_bounds__(256)
k_im2col_forward_f32(const float *__restrict__ x, float *__restrict__ y, Im2ColGeom g, float border_value, int p_tiles, int f_tiles)
{
    __shared__ float tile[kIm2ColTiles][32][33];
    const int tx = threadIdx.x, ty = threadIdx.y;
    int b = blockIdx.x;
    const int pt = b % p_tiles; b /= p_tiles;
    const int ft = b % f_tiles; b /= f_tiles;
    const int on = b;                                             // (c * filter_h + fy) * filter_w + fx
    const int fx = on % g.filter_w, fy = (on / g.filter_w) % g.filter_h, c = on / (g.filter_w * g.filter_h);
    const int P = g.out_w * g.out_h;
    const int p0 = pt * 32 * kIm2ColTiles, f0 = ft * 32;
    const int fi_r = f0 + tx;
    // the source node depends on the pixel only: one warp per tile works it out for 32 pixels (two integer divisions and the
    // border logic each), the loads below read it back as a broadcast
    __shared__ int s_src[kIm2ColTiles][32];
    if (ty < kIm2ColTiles) {
        const int p = p0 + 32 * ty + tx;
        s_src[ty][tx] = p < P ? im2col_source(g, c, fy, fx, p) : -2;
    }
    __syncthreads();
#pragma unroll
    for (int t = 0; t < kIm2ColTiles; ++t)
#pragma unroll
        for (int r = ty; r < 32; r += 8) {
            const int in = s_src[t][r];
            float v = border_value;
            if (in >= 0 && fi_r < g.in_frames) v = x[(size_t)in * g.in_fs + fi_r];
            tile[t][r][tx] = v;
        }
    __syncthreads();
    float *yrow = y + (size_t)on * g.out_fs;
#pragma unroll
    for (int t = 0; t < kIm2ColTiles; ++t)
#pragma unroll
        for (int r = ty; r < 32; r += 8) {
            const int fi = f0 + r, p = p0 + 32 * t + tx;
            if (p < P && fi < g.in_frames) yrow[(size_t)fi * P + p] = tile[t][tx][r];
        }
}

// Block = one channel x 32 input frames x 32 input pixels (q = y * W + x).  For every filter tap the threads of a warp read
// consecutive output pixels of one output frame row; the sums are turned through shared memory and written along frames.
__global__ void __launch_bounds__(256)
k_im2col_backward_f32(const float *__restrict__ dy, float *__restrict__ dx, Im2ColGeom g, int q_tiles, int f_tiles)
{
    __shared__ float tile[32][33];
    const int tx = threadIdx.x, ty = threadIdx.y;
    int b = blockIdx.x;
    const int qt = b % q_tiles; b /= q_tiles;
    const int ft = b % f_tiles; b /= f_tiles;
    const int c = b;
    const int Q = g.in_w * g.in_h, P = g.out_w * g.out_h;
    const int q = qt * 32 + tx;
    const int iy_limit = (g.out_h - 1) * g.y_stride, ix_limit = (g.out_w - 1) * g.x_stride;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (q < Q) {
        const int yy = q / g.in_w, xx = q % g.in_w;
        for (int fy = yy % g.y_stride; fy < g.filter_h; fy += g.y_stride) {
            const int iy = yy - fy + g.y_offset;
            if (iy < 0 || iy > iy_limit) continue;
            for (int fx = xx % g.x_stride; fx < g.filter_w; fx += g.x_stride) {
                const int ix = xx - fx + g.x_offset;
                if (ix < 0 || ix > ix_limit) continue;
                const int p  = (iy / g.y_stride) * g.out_w + ix / g.x_stride;
                const int on = (c * g.filter_h + fy) * g.filter_w + fx;
                const float *row = dy + (size_t)on * g.out_fs + p;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int fi = ft * 32 + ty + 8 * k;
                    if (fi < g.in_frames) acc[k] += row[(size_t)fi * P];
                }
            }
        }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) tile[ty + 8 * k][tx] = acc[k];            // [frame][pixel]
    __syncthreads();
#pragma unroll
    for (int r = ty; r < 32; r += 8) {
        const int qq = qt * 32 + r, fi = ft * 32 + tx;
        if (qq < Q && fi < g.in_frames) dx[(size_t)(c * Q + qq) * g.in_fs + fi] = tile[tx][r];
    }
}

// --------------------------------------------------------------------------------------------- Im2Col fp32, banded
// The two tile kernels above spend ~38 instructions per element on index arithmetic that does not depend on the frame (two
// integer divisions and the border logic per pixel, 64-bit offsets per element).  The banded kernels work that out once per
// CTA and reuse it over 32 frames and all filter taps:
//   block = one channel x one band of image rows x 32 input frames;
//   * forward: the band's input rows (with the filter's halo) are read once into shared memory, [pixel][frame], lanes along
//     frames; a table [tap][output pixel of the band] holds the shared-memory offset of the source pixel (or "border value", or a
//     global pixel index when a border mode maps outside the band); then every (tap, frame) pair is one contiguous run of the
//     output row, written by a warp with lanes along pixels -- one table read, one tile read, one store per element;
//   * backward: a table [tap][input pixel of the band] holds the output pixel that tap reads (the reference's own enumeration:
//     taps aligned with the pixel's position modulo the stride, in increasing order, include/bb/ConvolutionIm2Col.h:439-482);
//     a lane owns one input pixel and four frames, sums its taps in registers (reads along output pixels), and the band is turned
//     through shared memory so that the writes run along frames.
// kBandPitch = 33 keeps both the frame-major fill and the pixel-major read-out free of bank conflicts.
constexpr int kBandPitch = 33;
constexpr int kBandSmemLimit = 64 * 1024;

// Input pixel iy * in_w + ix (within a channel) read by output pixel (oy, ox) through tap (fy, fx), or -1 for the border value.
__device__ __forceinline__ int im2col_source_pixel(const Im2ColGeom &g, int fy, int fx, int oy, int ox)
{
    int iy = oy * g.y_stride - g.y_offset + fy;
    int ix = ox * g.x_stride - g.x_offset + fx;
    if (iy >= 0 && iy < g.in_h && ix >= 0 && ix < g.in_w) return iy * g.in_w + ix;
    if (border_remap(g.border_mode, ix, iy, g.in_w, g.in_h)) {
        if (iy >= 0 && iy < g.in_h && ix >= 0 && ix < g.in_w) return iy * g.in_w + ix;
    }
    return -1;
}

__global__ void __launch_bounds__(256)
k_im2col_forward_band_f32(const float *__restrict__ x, float *__restrict__ y, Im2ColGeom g, float border_value, int R, int rows_in, int bands,
                          int f_tiles)
{
    extern __shared__ __align__(16) unsigned char band_smem[];
    float *tile = reinterpret_cast<float *>(band_smem);                                   // [rows_in * in_w][kBandPitch]
    int *src = reinterpret_cast<int *>(tile + ((size_t)rows_in * g.in_w + 1) * kBandPitch);  // [taps][R * out_w], then [taps] flags
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int b = blockIdx.x;
    const int ft = b % f_tiles; b /= f_tiles;
    const int band = b % bands; b /= bands;
    const int c = b;
    const int oy0 = band * R, rows = min(R, g.out_h - oy0);
    const int npix = rows * g.out_w, pitch = R * g.out_w;
    const int iy0 = oy0 * g.y_stride - g.y_offset;                 // first input row an unremapped tap of the band reads
    const int f0 = ft * 32;
    const int taps = g.filter_h * g.filter_w;
    const int Q = g.in_h * g.in_w, P = g.out_h * g.out_w;

    // Source table: byte offset into the tile for every (tap, output pixel of the band).  A border pixel points at one extra tile
    // row that holds the border value in all 32 frames, so the copy loop needs no select; a source outside the band (only the
    // wrapping / reflecting border modes at a band edge) also points there for now and is remembered per tap in `patch` as
    // -2 - pixel, to be fetched from global memory afterwards.
    const int n_in = rows_in * g.in_w;
    int *patch = src + taps * pitch;                               // [taps]: 0, or 1 when the tap has sources outside the band
    if (threadIdx.x < taps) patch[threadIdx.x] = 0;
    __syncthreads();
    for (int pl = threadIdx.x; pl < npix; pl += 256) {
        const int oy = pl / g.out_w, ox = pl - oy * g.out_w;
        for (int fy = 0, tap = 0; fy < g.filter_h; ++fy)
            for (int fx = 0; fx < g.filter_w; ++fx, ++tap) {
                const int pix = im2col_source_pixel(g, fy, fx, oy0 + oy, ox);
                int s = n_in * (kBandPitch * 4);                   // the border row
                if (pix >= 0) {
                    const int local = pix - iy0 * g.in_w;          // in the band when 0 <= local < n_in
                    if (local >= 0 && local < n_in) s = local * (kBandPitch * 4);
                    else patch[tap] = 1;
                }
                src[tap * pitch + pl] = s;
            }
    }
    {
        const bool f_ok = f0 + lane < g.in_frames;
        const float *xc = x + (size_t)c * Q * g.in_fs + f0 + lane;
#pragma unroll 4
        for (int q = warp; q < n_in; q += 8) {
            const int pix = iy0 * g.in_w + q;
            float v = 0.0f;
            if (f_ok && pix >= 0 && pix < Q) v = xc[(size_t)pix * g.in_fs];
            tile[q * kBandPitch + lane] = v;
        }
        if (warp == 0) tile[n_in * kBandPitch + lane] = border_value;
    }
    __syncthreads();

    // (tap, frame) pairs: each is one contiguous run of an output row; an element is a table read, a tile read and a store.
    const int pairs = taps * 32;
    const unsigned char *tile_b = reinterpret_cast<const unsigned char *>(tile);
    for (int pr = warp; pr < pairs; pr += 8) {
        const int tap = pr >> 5, fl = pr & 31;                     // warp-uniform
        if (f0 + fl >= g.in_frames) continue;
        float *yrun = y + (size_t)(c * taps + tap) * g.out_fs + (size_t)(f0 + fl) * P + oy0 * g.out_w;
        float *yp = yrun + lane;
        const int *sp = src + tap * pitch + lane;
        const unsigned char *tp = tile_b + 4 * fl;
        int pl = lane;
        for (; pl + 96 < npix; pl += 128, sp += 128, yp += 128) {
            int sv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) sv[i] = sp[32 * i];
#pragma unroll
            for (int i = 0; i < 4; ++i) yp[32 * i] = *reinterpret_cast<const float *>(tp + sv[i]);
        }
        for (; pl < npix; pl += 32, sp += 32, yp += 32) yp[0] = *reinterpret_cast<const float *>(tp + sp[0]);
        if (patch[tap]) {
            const int fy = tap / g.filter_w, fx = tap - fy * g.filter_w;
            const float *xg = x + (size_t)c * Q * g.in_fs + f0 + fl;
            for (int q = lane; q < npix; q += 32) {
                const int oy = q / g.out_w, ox = q - oy * g.out_w;
                const int pix = im2col_source_pixel(g, fy, fx, oy0 + oy, ox);
                const int local = pix - iy0 * g.in_w;
                if (pix >= 0 && (local < 0 || local >= n_in)) yrun[q] = xg[(size_t)pix * g.in_fs];
            }
        }
    }
}

__global__ void __launch_bounds__(256)
k_im2col_backward_band_f32(const float *__restrict__ dy, float *__restrict__ dx, Im2ColGeom g, int R, int bands, int f_tiles)
{
    extern __shared__ __align__(16) unsigned char band_smem[];
    float *tile = reinterpret_cast<float *>(band_smem);                                   // [R * in_w][kBandPitch]
    int *src = reinterpret_cast<int *>(tile + (size_t)R * g.in_w * kBandPitch);            // [taps][R * in_w]: output pixel, or -1
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int b = blockIdx.x;
    const int ft = b % f_tiles; b /= f_tiles;
    const int band = b % bands; b /= bands;
    const int c = b;
    const int y0 = band * R, rows = min(R, g.in_h - y0);
    const int npix = rows * g.in_w, pitch = R * g.in_w;
    const int f0 = ft * 32;
    const int taps = g.filter_h * g.filter_w;
    const int Q = g.in_h * g.in_w, P = g.out_h * g.out_w;
    const int iy_limit = (g.out_h - 1) * g.y_stride, ix_limit = (g.out_w - 1) * g.x_stride;

    // the reference visits fy = yy % y_stride, + y_stride, ... and fx likewise; every other tap sends nothing to this pixel
    for (int ql = threadIdx.x; ql < npix; ql += 256) {
        const int yl = ql / g.in_w, xx = ql - yl * g.in_w, yy = y0 + yl;
        const bool ys1 = g.y_stride == 1, xs1 = g.x_stride == 1;
        const int ya = ys1 ? 0 : yy % g.y_stride, xa = xs1 ? 0 : xx % g.x_stride;
        for (int fy = 0, tap = 0; fy < g.filter_h; ++fy) {
            const int iy = yy - fy + g.y_offset;
            const bool y_ok = fy >= ya && (ys1 || (fy - ya) % g.y_stride == 0) && iy >= 0 && iy <= iy_limit;
            const int row = (ys1 ? iy : iy / g.y_stride) * g.out_w;
            for (int fx = 0; fx < g.filter_w; ++fx, ++tap) {
                const int ix = xx - fx + g.x_offset;
                const bool ok = y_ok && fx >= xa && (xs1 || (fx - xa) % g.x_stride == 0) && ix >= 0 && ix <= ix_limit;
                src[tap * pitch + ql] = ok ? row + (xs1 ? ix : ix / g.x_stride) : -1;
            }
        }
    }
    __syncthreads();

    // warp w owns frames f0 + w + 8 k, k = 0..3
    const float *base[4];
    bool ok[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int fi = f0 + warp + 8 * k;
        ok[k] = fi < g.in_frames;
        base[k] = dy + (size_t)c * taps * g.out_fs + (size_t)(ok[k] ? fi : 0) * P;
    }
    // Two pixels per lane and trip, three taps unrolled: 24 independent loads in flight per lane.  Every tap is loaded (a tap that
    // sends nothing reads element 0 of its row and adds zero) so that the loads do not wait for the table; x + 0 differs from x only
    // in the sign of a zero, which the final 0.0f + acc removes.
    for (int ql = lane; ql < npix; ql += 64) {
        const bool second = ql + 32 < npix;
        const int qb = second ? ql + 32 : ql;
        float acc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
#pragma unroll 3
        for (int tap = 0; tap < taps; ++tap) {
            const int sa = src[tap * pitch + ql], sb = src[tap * pitch + qb];
            const size_t row = (size_t)tap * g.out_fs;
            const size_t offa = row + (sa >= 0 ? sa : 0), offb = row + (sb >= 0 ? sb : 0);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float va = base[k][offa], vb = base[k][offb];
                acc[0][k] += (sa >= 0 && ok[k]) ? va : 0.0f;
                acc[1][k] += (sb >= 0 && ok[k]) ? vb : 0.0f;
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            tile[ql * kBandPitch + warp + 8 * k] = 0.0f + acc[0][k];
            if (second) tile[qb * kBandPitch + warp + 8 * k] = 0.0f + acc[1][k];
        }
    }
    __syncthreads();
    if (f0 + lane < g.in_frames) {
        float *dxc = dx + ((size_t)c * Q + (size_t)y0 * g.in_w) * g.in_fs + f0 + lane;
#pragma unroll 4
        for (int ql = warp; ql < npix; ql += 8) dxc[(size_t)ql * g.in_fs] = tile[ql * kBandPitch + lane];
    }
}

// --------------------------------------------------------------------------------------------- Im2Col bit
// P % 32 == 0: an output word is 32 consecutive pixels of one input frame.  A warp takes one group of 32 pixels (lane k owns pixel
// k and works out its source node once) and walks W input word columns (32 input frames each): lane k reads the word of its pixel,
// the transpose gives lane j the output word of input frame j.  A block covers up to 32 consecutive pixel groups, so each frame's
// words leave as one contiguous run, and W columns, so the source arithmetic (two divisions and the border logic per pixel) is
// spread over 32 W frames.
constexpr int kBitColumns = 8;

__global__ void __launch_bounds__(256)
k_im2col_forward_bit(const uint32_t *__restrict__ x, uint32_t *__restrict__ y, Im2ColGeom g, int groups, int g_tiles, int in_words, int w_tiles)
{
    __shared__ uint32_t tile[kBitColumns][32][33];                // [word column][input frame j][pixel group]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int b = blockIdx.x;
    const int gt = b % g_tiles; b /= g_tiles;
    const int wt = b % w_tiles; b /= w_tiles;
    const int on = b;
    const int fx = on % g.filter_w, fy = (on / g.filter_w) % g.filter_h, c = on / (g.filter_w * g.filter_h);
    const int g0 = gt * 32, gn = min(32, groups - g0);
    const int w0 = wt * kBitColumns, wn = min(kBitColumns, in_words - w0);
    const BitTranspose transpose(lane);
    for (int gl = warp; gl < gn; gl += 8) {
        const int in = im2col_source(g, c, fy, fx, (g0 + gl) * 32 + lane);
        const uint32_t *row = x + (size_t)(in >= 0 ? in : 0) * g.in_fs + w0;
        uint32_t v[kBitColumns];
#pragma unroll
        for (int wl = 0; wl < kBitColumns; ++wl) v[wl] = (in >= 0 && wl < wn) ? row[wl] : 0u;
        // (columns past the end of the row transpose zeros that nothing reads)
#pragma unroll
        for (int wl = 0; wl < kBitColumns; ++wl) tile[wl][lane][gl] = transpose(v[wl]);
    }
    __syncthreads();
    for (int r = warp; r < wn * 32; r += 8) {
        const int wl = r >> 5, j = r & 31;
        const int fi = (w0 + wl) * 32 + j;
        if (fi < g.in_frames && lane < gn) y[(size_t)on * g.out_fs + (size_t)fi * groups + g0 + lane] = tile[wl][j][lane];
    }
}

// Bit Im2Col for any geometry, by words.  The 32 input frames of one word column become 32 bit vectors over the channel's pixels
// (one 32 x 32 bit transpose per 32 pixels -- per input tile, not per filter tap).  Those 32 frames are exactly P consecutive
// output words of every tap, and an output word is the OR of a few masked 32-bit windows of such vectors: inside one image row
// the source pixels of consecutive output pixels are consecutive, so a window at bit offset (source pixel - output bit) yields all
// of them at once, and border pixels with their own offsets add a window each.  The windows of a word depend on the tap and on the
// word's position modulo the period (P / gcd(P, 32) words = 32 / gcd(P, 32) frames) only, so a small table built once per launch
// (k_im2col_bit_pieces) holds, per (tap, word of the period), up to kPieces entries {frame of the period, offset, mask}.
// A word that needs more windows than that (tiny images, strides above one) is marked and gathered bit by bit.
constexpr int kPieces = 12;
constexpr int kPieceBias = 64;                  // offsets are stored biased: they start at -31
constexpr unsigned kPieceOverflow = 0xffffffffu;

// One warp per (tap, word of the period); lane b owns output bit b, and the lanes whose (frame, offset) keys agree form one window.
__global__ void __launch_bounds__(256)
k_im2col_bit_pieces(Im2ColGeom g, int period_words, int2 *__restrict__ pieces)
{
    const int lane = threadIdx.x & 31;
    const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int taps = g.filter_h * g.filter_w;
    if (e >= taps * period_words) return;                          // warp-uniform
    const int tap = e / period_words, wp = e - tap * period_words;
    const int fy = tap / g.filter_w, fx = tap - fy * g.filter_w;
    const int P = g.out_h * g.out_w;
    const int o = 32 * wp + lane;
    const int dj = o / P, p = o - dj * P;
    const int oy = p / g.out_w, ox = p - oy * g.out_w;
    const int pix = im2col_source_pixel(g, fy, fx, oy, ox);        // -1: the border value of bit frames, 0
    const int key = pix >= 0 ? ((dj << 24) | (pix - lane + kPieceBias)) : -1;
    const unsigned same = __match_any_sync(0xffffffffu, key);      // the lanes of this lane's window
    const bool leader = pix >= 0 && (__ffs(same) - 1) == lane;
    const unsigned leaders = __ballot_sync(0xffffffffu, leader);
    const int n = __popc(leaders);
    int2 *out = pieces + (size_t)e * kPieces;
    if (n > kPieces) {
        if (lane == 0) out[0] = make_int2((int)kPieceOverflow, 0);
        return;
    }
    if (leader) out[__popc(leaders & ((1u << lane) - 1u))] = make_int2(key, (int)same);
    if (lane >= n && lane < kPieces) out[lane] = make_int2(0, 0);
}

__global__ void __launch_bounds__(256)
k_im2col_forward_bit_words(const uint32_t *__restrict__ x, uint32_t *__restrict__ y, Im2ColGeom g, const int2 *__restrict__ pieces, int period_words,
                           int period_frames, int qw, int in_words, long long out_words)
{
    extern __shared__ uint32_t bit_rows[];                        // [32 frames][qw + 2]: one zero word before and after every row
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wi = blockIdx.x % in_words, c = blockIdx.x / in_words;
    const int Q = g.in_h * g.in_w, P = g.out_h * g.out_w, pitch = qw + 2;
    const int taps = g.filter_h * g.filter_w;
    const BitTranspose transpose(lane);
    const bool frame_ok = wi * 32 + lane < g.in_frames;            // frames past the end read as zeros
    for (int k = warp; k < qw; k += 8) {
        const int pix = 32 * k + lane;
        const uint32_t v = pix < Q ? x[((size_t)c * Q + pix) * g.in_fs + wi] : 0u;
        const uint32_t t = transpose(v);
        bit_rows[lane * pitch + k + 1] = frame_ok ? t : 0u;
    }
    if (threadIdx.x < 64) bit_rows[(threadIdx.x >> 1) * pitch + ((threadIdx.x & 1) ? qw + 1 : 0)] = 0u;
    __syncthreads();

    // A lane keeps the windows of its word of the period (the first four in registers) and applies them to a run of up to eight
    // periods of the block's 32 frames; the warps share the (tap, run) units.
    const int periods = P / period_words;                          // = gcd(P, 32)
    const long long w_base = (long long)wi * P;
    const int w_limit = (int)min((long long)P, out_words - w_base);        // words of this block that exist (the last frames may not)
    const int run = min(8, periods), runs = (periods + run - 1) / run;
    for (int unit = warp; unit < taps * runs; unit += 8) {
        const int tap = unit / runs, np0 = (unit - tap * runs) * run, np1 = min(periods, np0 + run);
        uint32_t *yrow = y + (size_t)(c * taps + tap) * g.out_fs + w_base;
        for (int wp = lane; wp < period_words; wp += 32) {
            const int2 *pc = pieces + ((size_t)tap * period_words + wp) * kPieces;
            int2 e[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) e[k] = __ldg(pc + k);
            if ((unsigned)e[0].x == kPieceOverflow) {
                const int fy = tap / g.filter_w, fx = tap - fy * g.filter_w;
                for (int np = np0; np < np1; ++np) {
                    const int w = np * period_words + wp;
                    if (w >= w_limit) break;
                    const uint32_t *rows = bit_rows + np * period_frames * pitch;
                    uint32_t word = 0u;
                    for (int b = 0; b < 32; ++b) {
                        const int o = 32 * wp + b;
                        const int dj = o / P, p = o - dj * P;
                        const int oy = p / g.out_w, ox = p - oy * g.out_w;
                        const int pix = im2col_source_pixel(g, fy, fx, oy, ox);
                        if (pix >= 0) word |= ((rows[dj * pitch + 1 + (pix >> 5)] >> (pix & 31)) & 1u) << b;
                    }
                    yrow[w] = word;
                }
                continue;
            }
            // offsets inside the padded rows: word index and shift of every window; an unused window reads word 0 under an empty mask
            int at[4], sh[4];
            uint32_t mk[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int pos = (e[k].x & 0xffffff) - kPieceBias + 32;
                const bool used = e[k].y != 0;
                at[k] = used ? (e[k].x >> 24) * pitch + (pos >> 5) : 0;
                sh[k] = used ? (pos & 31) : 0;
                mk[k] = (uint32_t)e[k].y;
            }
            const bool more = e[3].y != 0 && __ldg(pc + 4).y != 0;
            for (int np = np0; np < np1; ++np) {
                const int w = np * period_words + wp;
                if (w >= w_limit) break;
                const uint32_t *rows = bit_rows + np * period_frames * pitch;
                uint32_t word = 0u;
#pragma unroll
                for (int k = 0; k < 4; ++k) word |= __funnelshift_r(rows[at[k]], rows[at[k] + 1], sh[k]) & mk[k];
                if (more) {
                    for (int k = 4; k < kPieces; ++k) {
                        const int2 f = __ldg(pc + k);
                        if (f.y == 0) break;
                        const int pos = (f.x & 0xffffff) - kPieceBias + 32;
                        const uint32_t *r = rows + (f.x >> 24) * pitch + (pos >> 5);
                        word |= __funnelshift_r(r[0], r[1], pos & 31) & (uint32_t)f.y;
                    }
                }
                yrow[w] = word;
            }
        }
    }
}

// Any P: one thread per output word gathers its 32 bits one by one.
__global__ void __launch_bounds__(256)
k_im2col_forward_bit_any(const uint32_t *__restrict__ x, uint32_t *__restrict__ y, Im2ColGeom g, int out_words, int out_nodes)
{
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long long)out_words * out_nodes) return;
    const int on = (int)(t / out_words), wo = (int)(t % out_words);
    const int fx = on % g.filter_w, fy = (on / g.filter_w) % g.filter_h, c = on / (g.filter_w * g.filter_h);
    const int P = g.out_w * g.out_h;
    const long long out_frames = (long long)g.in_frames * P;
    uint32_t word = 0;
    for (int k = 0; k < 32; ++k) {
        const long long fo = (long long)wo * 32 + k;
        if (fo >= out_frames) break;
        const int fi = (int)(fo / P), p = (int)(fo % P);
        const int in = im2col_source(g, c, fy, fx, p);
        if (in >= 0) word |= ((x[(size_t)in * g.in_fs + (fi >> 5)] >> (fi & 31)) & 1u) << k;
    }
    y[(size_t)on * g.out_fs + wo] = word;
}

// --------------------------------------------------------------------------------------------- Col2Im
// FORWARD: y[c * hw + xy][fo] = x[c][fo * hw + xy];  otherwise dx[c][fo * hw + xy] = dy[c * hw + xy][fo].
// Block = one channel x 64 pixels x 64 output frames, turned through shared memory: both sides move 256 contiguous bytes per row
// and every thread has 16 independent loads in flight before the barrier.  The image-side array is walked along frames, the
// column-side one along pixels.
constexpr int kCol2ImTile = 64;

template <bool FORWARD>
__global__ void __launch_bounds__(256)
k_col2im_f32(const float *__restrict__ src, float *__restrict__ dst, int hw, int out_frames, long long col_fs, long long img_fs, int xy_tiles,
             int f_tiles)
{
    __shared__ float tile[kCol2ImTile][kCol2ImTile + 1];
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
    int b = blockIdx.x;
    const int xt = b % xy_tiles; b /= xy_tiles;
    const int ft = b % f_tiles; b /= f_tiles;
    const int c = b;
    const int xy0 = xt * kCol2ImTile, f0 = ft * kCol2ImTile;
    if (FORWARD) {
#pragma unroll
        for (int r = ty; r < kCol2ImTile; r += 4) {               // r = frame, tx = pixel
            const int fo = f0 + r, xy = xy0 + tx;
            tile[r][tx] = (fo < out_frames && xy < hw) ? src[(size_t)c * col_fs + (size_t)fo * hw + xy] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int r = ty; r < kCol2ImTile; r += 4) {               // r = pixel, tx = frame
            const int xy = xy0 + r, fo = f0 + tx;
            if (fo < out_frames && xy < hw) dst[(size_t)(c * hw + xy) * img_fs + fo] = tile[tx][r];
        }
    } else {
#pragma unroll
        for (int r = ty; r < kCol2ImTile; r += 4) {               // r = pixel, tx = frame
            const int xy = xy0 + r, fo = f0 + tx;
            tile[r][tx] = (fo < out_frames && xy < hw) ? src[(size_t)(c * hw + xy) * img_fs + fo] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int r = ty; r < kCol2ImTile; r += 4) {               // r = frame, tx = pixel
            const int fo = f0 + r, xy = xy0 + tx;
            if (fo < out_frames && xy < hw) dst[(size_t)c * col_fs + (size_t)fo * hw + xy] = tile[tx][r];
        }
    }
}

// Warp = (channel, output word wo, group of 32 pixels): lane j takes, from the bit vector of output frame 32 wo + j (hw bits,
// starting at bit (32 wo + j) * hw of the channel's row, on no particular word boundary), the 32-bit window of the group's pixels;
// the transpose gives lane k the output word of pixel k.  A block takes 32 consecutive output words of the same pixel group, so
// every pixel's row receives one contiguous run.
__global__ void __launch_bounds__(256)
k_col2im_forward_bit(const uint32_t *__restrict__ x, uint32_t *__restrict__ y, int hw, int out_frames, long long in_fs, long long out_fs,
                     int groups, int w_tiles, int out_words, long long in_words)
{
    __shared__ uint32_t tile[32][33];                             // [pixel k][output word]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int b = blockIdx.x;
    const int wt = b % w_tiles; b /= w_tiles;
    const int gp = b % groups; b /= groups;
    const int c = b;
    const int w0 = wt * 32, wn = min(32, out_words - w0);
    const uint32_t *xr = x + (size_t)c * in_fs;
    const BitTranspose transpose(lane);
    for (int wl = warp; wl < wn; wl += 8) {
        const long long fo = (long long)(w0 + wl) * 32 + lane;
        uint32_t row = 0u;
        if (fo < out_frames) {
            const long long pos = fo * hw + 32 * gp;
            const long long wi = pos >> 5;
            const int sh = (int)(pos & 31);
            const uint32_t lo = xr[wi];
            const uint32_t hi = (sh != 0 && wi + 1 < in_words) ? xr[wi + 1] : 0u;       // (bits past the last frame belong to no pixel)
            row = __funnelshift_r(lo, hi, sh);
        }
        tile[lane][wl] = transpose(row);
    }
    __syncthreads();
    for (int k = warp; k < 32; k += 8)
        if (lane < wn && gp * 32 + k < hw) y[(size_t)(c * hw + gp * 32 + k) * out_fs + w0 + lane] = tile[k][lane];
}

// --------------------------------------------------------------------------------------------- MaxPooling
struct PoolGeom {
    int filter_h, filter_w, in_w, in_h, out_w, out_h, c_size, frames;
};

// One thread per (output node, V consecutive frames); grid.y walks the output nodes.  V = 4 (rows 16-byte aligned): 128-bit loads
// and stores, and the node arithmetic (three divisions per output node) is spread over four frames.
template <int V>
__global__ void __launch_bounds__(256)
k_maxpool_forward_f32(const float *__restrict__ x, float *__restrict__ y, int *__restrict__ argmax, PoolGeom g, long long fs)
{
    const int f = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (f >= g.frames) return;
    const bool full = f + V <= g.frames;
    for (int on = blockIdx.y; on < g.c_size * g.out_h * g.out_w; on += gridDim.y) {
        const int ox = on % g.out_w, oy = (on / g.out_w) % g.out_h, c = on / (g.out_w * g.out_h);
        float best[V];
        int am[V];
#pragma unroll
        for (int k = 0; k < V; ++k) { best[k] = -3.402823466e+38f; am[k] = 0; }      // std::numeric_limits<float>::lowest()
        int arg = 0;
        for (int fy = 0; fy < g.filter_h; ++fy) {
            const int iy = oy * g.filter_h + fy;
            if (iy >= g.in_h) break;
            for (int fx = 0; fx < g.filter_w; ++fx) {
                const int ix = ox * g.filter_w + fx;
                if (ix >= g.in_w) break;
                const float *p = x + (size_t)((c * g.in_h + iy) * g.in_w + ix) * fs + f;
                float v[V];
                if (V == 4) {              // inside the row's stride even when the last frames of the group do not exist
                    const float4 q = *reinterpret_cast<const float4 *>(p);
                    v[0] = q.x; v[1 % V] = q.y; v[2 % V] = q.z; v[3 % V] = q.w;
                } else {
                    v[0] = p[0];
                }
#pragma unroll
                for (int k = 0; k < V; ++k)
                    if (v[k] > best[k]) { best[k] = v[k]; am[k] = arg; }
                ++arg;
            }
        }
        float *yp = y + (size_t)on * fs + f;
        int *ap = argmax ? argmax + (size_t)on * fs + f : nullptr;
        if (V == 4 && full) {
            *reinterpret_cast<float4 *>(yp) = make_float4(best[0], best[1 % V], best[2 % V], best[3 % V]);
            if (ap) *reinterpret_cast<int4 *>(ap) = make_int4(am[0], am[1 % V], am[2 % V], am[3 % V]);
        } else {
#pragma unroll
            for (int k = 0; k < V; ++k)
                if (f + k < g.frames) { yp[k] = best[k]; if (ap) ap[k] = am[k]; }
        }
    }
}

__global__ void __launch_bounds__(256)
k_maxpool_forward_bit(const uint32_t *__restrict__ x, uint32_t *__restrict__ y, PoolGeom g, long long fs, int words)
{
    const int w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w >= words) return;
    for (int on = blockIdx.y; on < g.c_size * g.out_h * g.out_w; on += gridDim.y) {
        const int ox = on % g.out_w, oy = (on / g.out_w) % g.out_h, c = on / (g.out_w * g.out_h);
        uint32_t m = 0;
        for (int fy = 0; fy < g.filter_h; ++fy) {
            const int iy = oy * g.filter_h + fy;
            if (iy >= g.in_h) break;
            for (int fx = 0; fx < g.filter_w; ++fx) {
                const int ix = ox * g.filter_w + fx;
                if (ix >= g.in_w) break;
                m |= x[(size_t)((c * g.in_h + iy) * g.in_w + ix) * fs + w];
            }
        }
        y[(size_t)on * fs + w] = m;
    }
}

// XBITS = false: routed by argmax; XBITS = true: the first set input bit of the window takes the gradient.  V as in the forward.
template <bool XBITS, int V>
__global__ void __launch_bounds__(256)
k_maxpool_backward(const void *__restrict__ sel, const float *__restrict__ dy, float *__restrict__ dx, PoolGeom g, long long sel_fs, long long fs)
{
    const int f = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (f >= g.frames) return;
    const bool full = f + V <= g.frames;
    for (int on = blockIdx.y; on < g.c_size * g.out_h * g.out_w; on += gridDim.y) {
        const int ox = on % g.out_w, oy = (on / g.out_w) % g.out_h, c = on / (g.out_w * g.out_h);
        float grad[V];
        int am[V];
        if (V == 4) {
            const float4 q = *reinterpret_cast<const float4 *>(dy + (size_t)on * fs + f);
            grad[0] = q.x; grad[1 % V] = q.y; grad[2 % V] = q.z; grad[3 % V] = q.w;
            if (!XBITS) {
                const int4 a = *reinterpret_cast<const int4 *>(static_cast<const int *>(sel) + (size_t)on * sel_fs + f);
                am[0] = a.x; am[1 % V] = a.y; am[2 % V] = a.z; am[3 % V] = a.w;
            }
        } else {
            grad[0] = dy[(size_t)on * fs + f];
            am[0] = XBITS ? 0 : static_cast<const int *>(sel)[(size_t)on * sel_fs + f];
        }
        int arg = 0;
        for (int fy = 0; fy < g.filter_h; ++fy) {
            const int iy = oy * g.filter_h + fy;
            if (iy >= g.in_h) break;
            for (int fx = 0; fx < g.filter_w; ++fx) {
                const int ix = ox * g.filter_w + fx;
                if (ix >= g.in_w) break;
                const size_t in = (size_t)((c * g.in_h + iy) * g.in_w + ix);
                float out[V];
                if (XBITS) {
                    const uint32_t word = static_cast<const uint32_t *>(sel)[in * sel_fs + (f >> 5)];      // V frames from a multiple of V: one word
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        const bool bit = (word >> ((f + k) & 31)) & 1u;
                        out[k] = bit ? grad[k] : 0.0f;
                        if (bit) grad[k] = 0.0f;
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < V; ++k) out[k] = (arg == am[k]) ? grad[k] : 0.0f;
                    ++arg;
                }
                float *dp = dx + in * fs + f;
                if (V == 4 && full) {
                    *reinterpret_cast<float4 *>(dp) = make_float4(out[0], out[1 % V], out[2 % V], out[3 % V]);
                } else {
#pragma unroll
                    for (int k = 0; k < V; ++k)
                        if (f + k < g.frames) dp[k] = out[k];
                }
            }
        }
    }
}

// Rows per band of the banded Im2Col kernels: at most `fit` (what shared memory holds) and at most 8, halved while the grid has fewer
// than four blocks per SM.  Measured on B200 (32 channels of 32 x 32, 256 frames, 3 x 3): forward 0.161 / 0.105 / 0.077 / 0.076 /
// 0.104 ms at 1 / 2 / 4 / 8 / 10 rows -- short bands write short runs per frame, tall ones leave too few blocks.
int band_rows_for_occupancy(int fit, int rows_total, long long other_blocks)
{
    int R = fit < rows_total ? fit : rows_total;
    if (R > 8) R = 8;
    const long long want = 4LL * device_info().sm_count;
    while (R > 1 && other_blocks * ((rows_total + R - 1) / R) < want) R = (R + 1) / 2;
    return R;
}

int check_im2col(const void *a, const void *b, int x_stride, int y_stride, int in_frames, long long in_fs, int in_w, int in_h, int in_c, int out_w,
                 int out_h, long long out_fs, int filter_w, int filter_h, int frames_per_unit_in, int frames_per_unit_out)
{
    BB200_REQUIRE_PTR(a); BB200_REQUIRE_PTR(b);
    BB200_REQUIRE(x_stride >= 1 && y_stride >= 1 && in_frames >= 0 && in_w >= 1 && in_h >= 1 && in_c >= 0 && out_w >= 0 && out_h >= 0 &&
                  filter_w >= 1 && filter_h >= 1, BBCU_ERR_BAD_SIZE);
    const long long out_frames = (long long)in_frames * out_w * out_h;
    BB200_REQUIRE(out_frames < (1LL << 31) && (long long)in_c * in_h * in_w < (1LL << 31) && (long long)in_c * filter_h * filter_w < (1LL << 31),
                  BBCU_ERR_TOO_LARGE);
    BB200_REQUIRE(in_fs * frames_per_unit_in >= in_frames && out_fs * frames_per_unit_out >= out_frames, BBCU_ERR_BAD_STRIDE);
    return BBCU_OK;
}

Im2ColGeom make_geom(int x_stride, int y_stride, int x_offset, int y_offset, int in_frames, long long in_fs, int in_w, int in_h, int in_c, int out_w,
                     int out_h, long long out_fs, int filter_w, int filter_h, int border_mode)
{
    Im2ColGeom g;
    g.x_stride = x_stride; g.y_stride = y_stride; g.x_offset = x_offset; g.y_offset = y_offset;
    g.in_w = in_w; g.in_h = in_h; g.in_c = in_c; g.out_w = out_w; g.out_h = out_h; g.filter_w = filter_w; g.filter_h = filter_h;
    g.border_mode = border_mode; g.in_frames = in_frames; g.in_fs = in_fs; g.out_fs = out_fs;
    return g;
}

int check_pool(const void *a, const void *b, int fh, int fw, int in_w, int in_h, int out_w, int out_h, int c_size, int frames)
{
    BB200_REQUIRE_PTR(a); BB200_REQUIRE_PTR(b);
    BB200_REQUIRE(fh >= 1 && fw >= 1 && in_w >= 1 && in_h >= 1 && c_size >= 0 && frames >= 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE(out_w == (in_w + fw - 1) / fw && out_h == (in_h + fh - 1) / fh, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE((long long)c_size * in_h * in_w < (1LL << 31), BBCU_ERR_TOO_LARGE);
    return BBCU_OK;
}

PoolGeom make_pool(int fh, int fw, int in_w, int in_h, int out_w, int out_h, int c_size, int frames)
{
    PoolGeom g;
    g.filter_h = fh; g.filter_w = fw; g.in_w = in_w; g.in_h = in_h; g.out_w = out_w; g.out_h = out_h; g.c_size = c_size; g.frames = frames;
    return g;
}

inline unsigned grid_y(long long nodes) { return (unsigned)(nodes < 65535 ? (nodes > 0 ? nodes : 1) : 65535); }

}   // namespace
}   // namespace bb200

using namespace bb200;

// ----------------------------------------------------------------------------------------------------- Im2Col
extern "C" int bbcu_fp32_Im2Col_Forward(const float *dev_x_buf, float *dev_y_buf, int x_stride, int y_stride, int x_offset, int y_offset,
                                        int input_frame_size, int input_frame_stride, int input_w_size, int input_h_size, int input_c_size,
                                        int output_w_size, int output_h_size, int output_frame_stride, int filter_w_size, int filter_h_size,
                                        int border_mode, float border_value, bbcu_stream_t stream)
{
    int rc = check_im2col(dev_x_buf, dev_y_buf, x_stride, y_stride, input_frame_size, input_frame_stride, input_w_size, input_h_size, input_c_size,
                          output_w_size, output_h_size, output_frame_stride, filter_w_size, filter_h_size, 1, 1);
    if (rc) return rc;
    const long long P = (long long)output_w_size * output_h_size, out_nodes = (long long)input_c_size * filter_h_size * filter_w_size;
    if (P == 0 || input_frame_size == 0 || out_nodes == 0) return BBCU_OK;
    const Im2ColGeom g = make_geom(x_stride, y_stride, x_offset, y_offset, input_frame_size, input_frame_stride, input_w_size, input_h_size,
                                   input_c_size, output_w_size, output_h_size, output_frame_stride, filter_w_size, filter_h_size, border_mode);
    const int f_tiles = (input_frame_size + 31) / 32;
    {
        // banded kernel: the widest band of output rows whose input rows and source table fit the shared-memory budget
        const int taps = filter_h_size * filter_w_size;
        auto rows_in_of = [&](int R) { return (long long)(R - 1) * y_stride + filter_h_size; };
        auto smem_of = [&](int R) { return ((rows_in_of(R) * input_w_size + 1) * kBandPitch + (long long)taps * R * output_w_size + taps) * 4; };
        // smem_of(R) = R * per_row + fixed
        const long long per_row = ((long long)y_stride * input_w_size * kBandPitch + (long long)taps * output_w_size) * 4;
        const long long fixed = ((long long)(filter_h_size - y_stride) * input_w_size * kBandPitch + kBandPitch + taps) * 4;
        long long fit = (kBandSmemLimit - fixed) / per_row;
        if (fit > output_h_size) fit = output_h_size;
        while (fit >= 1 && smem_of((int)fit) > kBandSmemLimit) --fit;
        int R = fit >= 1 ? (int)fit : 0;
        if (R > 0) {
            R = band_rows_for_occupancy(R, output_h_size, (long long)input_c_size * f_tiles);
            const int bands = (output_h_size + R - 1) / R;
            const long long blocks = (long long)input_c_size * bands * f_tiles;
            BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
            const int smem = (int)smem_of(R);
            BB200_CUDA(cudaFuncSetAttribute(k_im2col_forward_band_f32, cudaFuncAttributeMaxDynamicSharedMemorySize, kBandSmemLimit));
            k_im2col_forward_band_f32<<<(unsigned)blocks, 256, smem, as_stream(stream)>>>(dev_x_buf, dev_y_buf, g, border_value, R, (int)rows_in_of(R),
                                                                                       bands, f_tiles);
            return launch_status();
        }
    }
    // images too wide for a band in shared memory: 32 x 32 tile transposes
    const int p_tiles = (int)((P + 32 * kIm2ColTiles - 1) / (32 * kIm2ColTiles));
    const long long blocks = out_nodes * p_tiles * f_tiles;
    BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
    k_im2col_forward_f32<<<(unsigned)blocks, dim3(32, 8), 0, as_stream(stream)>>>(dev_x_buf, dev_y_buf, g, border_value, p_tiles, f_tiles);
    return launch_status();
}

extern "C" int bbcu_bit_Im2Col_Forward(const int *dev_x_buf, int *dev_y_buf, int x_stride, int y_stride, int x_offset, int y_offset,
                                       int input_frame_size, int input_frame_stride, int input_w_size, int input_h_size, int input_c_size,
                                       int output_w_size, int output_h_size, int output_frame_stride, int filter_w_size, int filter_h_size,
                                       int border_mode, bbcu_stream_t stream)
{
    int rc = check_im2col(dev_x_buf, dev_y_buf, x_stride, y_stride, input_frame_size, input_frame_stride, input_w_size, input_h_size, input_c_size,
                          output_w_size, output_h_size, output_frame_stride, filter_w_size, filter_h_size, 32, 32);
    if (rc) return rc;
    const long long P = (long long)output_w_size * output_h_size, out_nodes = (long long)input_c_size * filter_h_size * filter_w_size;
    if (P == 0 || input_frame_size == 0 || out_nodes == 0) return BBCU_OK;
    const Im2ColGeom g = make_geom(x_stride, y_stride, x_offset, y_offset, input_frame_size, input_frame_stride, input_w_size, input_h_size,
                                   input_c_size, output_w_size, output_h_size, output_frame_stride, filter_w_size, filter_h_size, border_mode);
    const uint32_t *x = reinterpret_cast<const uint32_t *>(dev_x_buf);
    uint32_t *y = reinterpret_cast<uint32_t *>(dev_y_buf);
    {
        // by words: the piece table lives in the stream's scratch; images whose 32 bit rows do not fit shared memory, or a heap
        // that declines the table, take the kernels below
        int gcd = 32;
        while (P % gcd != 0) gcd >>= 1;
        const int period_words = (int)(P / gcd), period_frames = 32 / gcd;
        const int taps = filter_h_size * filter_w_size, in_words = (input_frame_size + 31) / 32;
        const int qw = (input_w_size * input_h_size + 31) / 32;
        const size_t smem = (size_t)32 * (qw + 2) * 4, table_bytes = (size_t)taps * period_words * kPieces * sizeof(int2);
        const long long blocks = (long long)input_c_size * in_words;
        if (smem <= 48 * 1024 && table_bytes <= (64u << 20) && blocks < (1LL << 31)) {
            int2 *pieces = static_cast<int2 *>(stream_scratch(as_stream(stream), table_bytes, 2));
            if (pieces != nullptr) {
                const int entries = taps * period_words;
                k_im2col_bit_pieces<<<(entries + 7) / 8, 256, 0, as_stream(stream)>>>(g, period_words, pieces);
                BB200_CUDA(cudaPeekAtLastError());
                const long long out_words = ((long long)input_frame_size * P + 31) / 32;
                k_im2col_forward_bit_words<<<(unsigned)blocks, 256, smem, as_stream(stream)>>>(x, y, g, pieces, period_words, period_frames, qw, in_words,
                                                                                              out_words);
                return launch_status();
            }
        }
    }
    if (P % 32 == 0) {
        const int groups = (int)(P / 32), g_tiles = (groups + 31) / 32, in_words = (input_frame_size + 31) / 32;
        const int w_tiles = (in_words + kBitColumns - 1) / kBitColumns;
        const long long blocks = out_nodes * w_tiles * g_tiles;
        BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
        k_im2col_forward_bit<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(x, y, g, groups, g_tiles, in_words, w_tiles);
    } else {
        const long long out_words = ((long long)input_frame_size * P + 31) / 32;
        const long long blocks = (out_words * out_nodes + 255) / 256;
        BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
        k_im2col_forward_bit_any<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(x, y, g, (int)out_words, (int)out_nodes);
    }
    return launch_status();
}

extern "C" int bbcu_fp32_Im2Col_Backward(const float *dev_dy_buf, float *dev_dx_buf, int x_stride, int y_stride, int x_offset, int y_offset,
                                         int input_frame_size, int input_frame_stride, int input_w_size, int input_h_size, int input_c_size,
                                         int output_w_size, int output_h_size, int output_frame_stride, int filter_w_size, int filter_h_size,
                                         bbcu_stream_t stream)
{
    int rc = check_im2col(dev_dy_buf, dev_dx_buf, x_stride, y_stride, input_frame_size, input_frame_stride, input_w_size, input_h_size,
                          input_c_size, output_w_size, output_h_size, output_frame_stride, filter_w_size, filter_h_size, 1, 1);
    if (rc) return rc;
    if (input_c_size == 0 || input_frame_size == 0) return BBCU_OK;
    const Im2ColGeom g = make_geom(x_stride, y_stride, x_offset, y_offset, input_frame_size, input_frame_stride, input_w_size, input_h_size,
                                   input_c_size, output_w_size, output_h_size, output_frame_stride, filter_w_size, filter_h_size, kBorderConstant);
    const int f_tiles = (input_frame_size + 31) / 32;
    {
        const int taps = filter_h_size * filter_w_size;
        const long long per_row = (long long)input_w_size * (kBandPitch + taps) * 4;
        int R = (int)(kBandSmemLimit / per_row);
        if (R > input_h_size) R = input_h_size;
        if (R > 0 && output_w_size > 0 && output_h_size > 0) {        // (the banded kernel reads element 0 of a row for a tap that sends nothing)
            R = band_rows_for_occupancy(R, input_h_size, (long long)input_c_size * f_tiles);
            const int bands = (input_h_size + R - 1) / R;
            const long long blocks = (long long)input_c_size * bands * f_tiles;
            BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
            BB200_CUDA(cudaFuncSetAttribute(k_im2col_backward_band_f32, cudaFuncAttributeMaxDynamicSharedMemorySize, kBandSmemLimit));
            k_im2col_backward_band_f32<<<(unsigned)blocks, 256, (int)(per_row * R), as_stream(stream)>>>(dev_dy_buf, dev_dx_buf, g, R, bands, f_tiles);
            return launch_status();
        }
    }
    const int q_tiles = (input_w_size * input_h_size + 31) / 32;
    const long long blocks = (long long)input_c_size * q_tiles * f_tiles;
    BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
    k_im2col_backward_f32<<<(unsigned)blocks, dim3(32, 8), 0, as_stream(stream)>>>(dev_dy_buf, dev_dx_buf, g, q_tiles, f_tiles);
    return launch_status();
}

// ----------------------------------------------------------------------------------------------------- Col2Im
static int check_col2im(const void *a, const void *b, int w, int h, int c, long long col_fs, int out_frames, long long img_fs, int unit)
{
    BB200_REQUIRE_PTR(a); BB200_REQUIRE_PTR(b);
    BB200_REQUIRE(w >= 1 && h >= 1 && c >= 0 && out_frames >= 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE((long long)out_frames * w * h < (1LL << 31) && (long long)c * w * h < (1LL << 31), BBCU_ERR_TOO_LARGE);
    BB200_REQUIRE(col_fs * unit >= (long long)out_frames * w * h && img_fs * unit >= out_frames, BBCU_ERR_BAD_STRIDE);
    return BBCU_OK;
}

template <bool FORWARD>
static int col2im_f32(const float *src, float *dst, int w, int h, int c, int col_fs, int out_frames, int img_fs, cudaStream_t st)
{
    int rc = check_col2im(src, dst, w, h, c, col_fs, out_frames, img_fs, 1);
    if (rc) return rc;
    if (c == 0 || out_frames == 0) return BBCU_OK;
    const int hw = w * h, xy_tiles = (hw + kCol2ImTile - 1) / kCol2ImTile, f_tiles = (out_frames + kCol2ImTile - 1) / kCol2ImTile;
    const long long blocks = (long long)c * xy_tiles * f_tiles;
    BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
    k_col2im_f32<FORWARD><<<(unsigned)blocks, 256, 0, st>>>(src, dst, hw, out_frames, col_fs, img_fs, xy_tiles, f_tiles);
    return launch_status();
}

extern "C" int bbcu_fp32_Col2Im_Forward(const float *dev_x_buf, float *dev_y_buf, int w_size, int h_size, int c_size, int input_frame_stride,
                                        int output_frame_size, int output_frame_stride, bbcu_stream_t stream)
{
    return col2im_f32<true>(dev_x_buf, dev_y_buf, w_size, h_size, c_size, input_frame_stride, output_frame_size, output_frame_stride,
                            as_stream(stream));
}

extern "C" int bbcu_fp32_Col2Im_Backward(const float *dev_dy_buf, float *dev_dx_buf, int w_size, int h_size, int c_size, int input_frame_stride,
                                         int output_frame_size, int output_frame_stride, bbcu_stream_t stream)
{
    return col2im_f32<false>(dev_dy_buf, dev_dx_buf, w_size, h_size, c_size, input_frame_stride, output_frame_size, output_frame_stride,
                             as_stream(stream));
}

extern "C" int bbcu_bit_Col2Im_Forward(const int *dev_x_buf, int *dev_y_buf, int w_size, int h_size, int c_size, int input_frame_stride,
                                       int output_frame_size, int output_frame_stride, bbcu_stream_t stream)
{
    int rc = check_col2im(dev_x_buf, dev_y_buf, w_size, h_size, c_size, input_frame_stride, output_frame_size, output_frame_stride, 32);
    if (rc) return rc;
    if (c_size == 0 || output_frame_size == 0) return BBCU_OK;
    const uint32_t *x = reinterpret_cast<const uint32_t *>(dev_x_buf);
    uint32_t *y = reinterpret_cast<uint32_t *>(dev_y_buf);
    const int hw = w_size * h_size, out_words = (output_frame_size + 31) / 32;
    const int groups = (hw + 31) / 32, w_tiles = (out_words + 31) / 32;
    const long long in_words = ((long long)output_frame_size * hw + 31) / 32;
    const long long blocks = (long long)c_size * groups * w_tiles;
    BB200_REQUIRE(blocks < (1LL << 31), BBCU_ERR_TOO_LARGE);
    k_col2im_forward_bit<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(x, y, hw, output_frame_size, input_frame_stride, output_frame_stride, groups,
                                                                         w_tiles, out_words, in_words);
    return launch_status();
}

// ----------------------------------------------------------------------------------------------------- MaxPooling
extern "C" int bbcu_fp32_MaxPooling_Forward(const float *dev_x_buf, float *dev_y_buf, int *dev_argmax_buf, int filter_h_size, int filter_w_size,
                                            int input_w_size, int input_h_size, int output_w_size, int output_h_size, int c_size, int frame_size,
                                            int frame_stride, bbcu_stream_t stream)
{
    int rc = check_pool(dev_x_buf, dev_y_buf, filter_h_size, filter_w_size, input_w_size, input_h_size, output_w_size, output_h_size, c_size, frame_size);
    if (rc) return rc;
    BB200_REQUIRE(frame_stride >= frame_size, BBCU_ERR_BAD_STRIDE);
    if (c_size == 0 || frame_size == 0) return BBCU_OK;
    const PoolGeom g = make_pool(filter_h_size, filter_w_size, input_w_size, input_h_size, output_w_size, output_h_size, c_size, frame_size);
    const bool vec = frame_stride % 4 == 0 && ((reinterpret_cast<uintptr_t>(dev_x_buf) | reinterpret_cast<uintptr_t>(dev_y_buf) |
                                               reinterpret_cast<uintptr_t>(dev_argmax_buf)) & 15) == 0;
    const int per = vec ? 4 : 1;
    dim3 grid(((frame_size + per - 1) / per + 255) / 256, grid_y((long long)c_size * output_h_size * output_w_size));
    if (vec) k_maxpool_forward_f32<4><<<grid, 256, 0, as_stream(stream)>>>(dev_x_buf, dev_y_buf, dev_argmax_buf, g, frame_stride);
    else     k_maxpool_forward_f32<1><<<grid, 256, 0, as_stream(stream)>>>(dev_x_buf, dev_y_buf, dev_argmax_buf, g, frame_stride);
    return launch_status();
}

extern "C" int bbcu_bit_MaxPooling_Forward(const int *dev_x_buf, int *dev_y_buf, int filter_h_size, int filter_w_size, int input_w_size,
                                           int input_h_size, int output_w_size, int output_h_size, int c_size, int frame_size, int frame_stride,
                                           bbcu_stream_t stream)
{
    int rc = check_pool(dev_x_buf, dev_y_buf, filter_h_size, filter_w_size, input_w_size, input_h_size, output_w_size, output_h_size, c_size, frame_size);
    if (rc) return rc;
    BB200_REQUIRE((long long)frame_stride * 32 >= frame_size, BBCU_ERR_BAD_STRIDE);
    if (c_size == 0 || frame_size == 0) return BBCU_OK;
    const PoolGeom g = make_pool(filter_h_size, filter_w_size, input_w_size, input_h_size, output_w_size, output_h_size, c_size, frame_size);
    const int words = (frame_size + 31) / 32;
    dim3 grid((words + 255) / 256, grid_y((long long)c_size * output_h_size * output_w_size));
    k_maxpool_forward_bit<<<grid, 256, 0, as_stream(stream)>>>(reinterpret_cast<const uint32_t *>(dev_x_buf), reinterpret_cast<uint32_t *>(dev_y_buf), g,
                                                              frame_stride, words);
    return launch_status();
}

extern "C" int bbcu_fp32_MaxPooling_Backward(const int *dev_argmax_buf, const float *dev_dy_buf, float *dev_dx_buf, int filter_h_size,
                                             int filter_w_size, int input_w_size, int input_h_size, int output_w_size, int output_h_size, int c_size,
                                             int frame_size, int frame_stride, bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(dev_argmax_buf);
    int rc = check_pool(dev_dy_buf, dev_dx_buf, filter_h_size, filter_w_size, input_w_size, input_h_size, output_w_size, output_h_size, c_size, frame_size);
    if (rc) return rc;
    BB200_REQUIRE(frame_stride >= frame_size, BBCU_ERR_BAD_STRIDE);
    if (c_size == 0 || frame_size == 0) return BBCU_OK;
    const PoolGeom g = make_pool(filter_h_size, filter_w_size, input_w_size, input_h_size, output_w_size, output_h_size, c_size, frame_size);
    const bool vec = frame_stride % 4 == 0 && ((reinterpret_cast<uintptr_t>(dev_argmax_buf) | reinterpret_cast<uintptr_t>(dev_dy_buf) |
                                               reinterpret_cast<uintptr_t>(dev_dx_buf)) & 15) == 0;
    const int per = vec ? 4 : 1;
    dim3 grid(((frame_size + per - 1) / per + 255) / 256, grid_y((long long)c_size * output_h_size * output_w_size));
    if (vec) k_maxpool_backward<false, 4><<<grid, 256, 0, as_stream(stream)>>>(dev_argmax_buf, dev_dy_buf, dev_dx_buf, g, frame_stride, frame_stride);
    else     k_maxpool_backward<false, 1><<<grid, 256, 0, as_stream(stream)>>>(dev_argmax_buf, dev_dy_buf, dev_dx_buf, g, frame_stride, frame_stride);
    return launch_status();
}

extern "C" int bbcu_bit_fp32_MaxPooling_Backward(const int *dev_x_buf, const float *dev_dy_buf, float *dev_dx_buf, int filter_h_size,
                                                 int filter_w_size, int input_w_size, int input_h_size, int output_w_size, int output_h_size,
                                                 int c_size, int frame_size, int forward_frame_stride, int backward_frame_stride,
                                                 bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(dev_x_buf);
    int rc = check_pool(dev_dy_buf, dev_dx_buf, filter_h_size, filter_w_size, input_w_size, input_h_size, output_w_size, output_h_size, c_size, frame_size);
    if (rc) return rc;
    BB200_REQUIRE(backward_frame_stride >= frame_size && (long long)forward_frame_stride * 32 >= frame_size, BBCU_ERR_BAD_STRIDE);
    if (c_size == 0 || frame_size == 0) return BBCU_OK;
    const PoolGeom g = make_pool(filter_h_size, filter_w_size, input_w_size, input_h_size, output_w_size, output_h_size, c_size, frame_size);
    const bool vec = backward_frame_stride % 4 == 0 && ((reinterpret_cast<uintptr_t>(dev_dy_buf) | reinterpret_cast<uintptr_t>(dev_dx_buf)) & 15) == 0;
    const int per = vec ? 4 : 1;
    dim3 grid(((frame_size + per - 1) / per + 255) / 256, grid_y((long long)c_size * output_h_size * output_w_size));
    if (vec) k_maxpool_backward<true, 4><<<grid, 256, 0, as_stream(stream)>>>(dev_x_buf, dev_dy_buf, dev_dx_buf, g, forward_frame_stride, backward_frame_stride);
    else     k_maxpool_backward<true, 1><<<grid, 256, 0, as_stream(stream)>>>(dev_x_buf, dev_dy_buf, dev_dx_buf, g, forward_frame_stride, backward_frame_stride);
    return launch_status();
}
