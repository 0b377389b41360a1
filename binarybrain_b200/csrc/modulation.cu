// Binary modulation around a LUT network: RealToBinary turns one fp32 frame into frame_mod
// bit frames by comparing against a threshold per output frame, BinaryToReal integrates bit frames back into fp32.
//
// Semantics follow the reference's CPU branches:
//   RealToBinary  include/bb/RealToBinary.h:309-345 (deterministic thresholds), :352-398 (thresholds from a value generator;
//                 here the caller passes them, because the reference draws them on the host)
//   BinaryToReal  include/bb/BinaryToReal.h:247-276 (forward), :312-330 (backward)
#include "common.cuh"

namespace bb200 {

// One warp per (output node, 32 input frames x frame_mod output frames): lane = input frame; each lane produces its
// frame_mod bits, which land in consecutive output frames  f_in * frame_mod + f.
__global__ void __launch_bounds__(256)
k_real_to_binary_bit(const float *__restrict__ x, uint32_t *y, const float *__restrict__ th, unsigned depth_mod, unsigned frame_mod, float lo,
                     float hi, unsigned point_size, unsigned x_frame_size, long long xs, long long ys, long long ths, unsigned out_nodes)
{
    const unsigned node = blockIdx.y;                                  // output node = (input_depth * depth_mod + d) * point_size + p
    const unsigned of = blockIdx.x * blockDim.x + threadIdx.x;         // output frame
    const unsigned out_frames = x_frame_size * frame_mod;
    const bool live = of < out_frames && node < out_nodes;
    bool bit = false;
    if (live) {
        const unsigned p = node % point_size, od = node / point_size;
        const unsigned d = od % depth_mod, in_depth = od / depth_mod;
        const unsigned in_node = in_depth * point_size + p;
        const unsigned fi = of / frame_mod, f = of % frame_mod;
        const float depth_step = 1.0f / (float)depth_mod, frame_step = 1.0f / (float)frame_mod;
        float v = (x[(size_t)in_node * xs + fi] - lo) * (1.0f / (hi - lo));
        v = (v - (float)d * depth_step) * (float)depth_mod;
        if (th != nullptr) {
            bit = v > th[(size_t)in_node * ths + of];
        } else {
            v = (v - (float)f * frame_step) * (float)frame_mod;
            v = fmaxf(0.0f, fminf(1.0f, v));
            bit = v > 0.5f;
        }
    }
    const unsigned word = __ballot_sync(0xffffffffu, bit);
    if ((threadIdx.x & 31) == 0 && of < out_frames && node < out_nodes) y[(size_t)node * ys + (of >> 5)] = word;
}

// y[f][n] = mean over i < node_mux, j < frame_mux of bit x[f * frame_mux + j][n + i * y_nodes]
template <bool XBIT>
__global__ void k_binary_to_real_forward(const void *x, float *y, int node_mux, int frame_mux, int y_nodes, long long xs, int y_frames, long long ys)
{
    const int f = blockIdx.x * blockDim.x + threadIdx.x;
    const int n = blockIdx.y;
    if (f >= y_frames) return;
    float sum = 0.0f;
    for (int i = 0; i < node_mux; ++i) {
        const size_t row = (size_t)(n + i * y_nodes) * xs;
        for (int j = 0; j < frame_mux; ++j) {
            const long long xf = (long long)f * frame_mux + j;
            if (XBIT) sum += (float)((static_cast<const uint32_t *>(x)[row + (xf >> 5)] >> (xf & 31)) & 1u);
            else      sum += static_cast<const float *>(x)[row + xf] > 0.0f ? 1.0f : 0.0f;
        }
    }
    y[(size_t)n * ys + f] = sum / (float)(node_mux * frame_mux);
}

// dx[f * frame_mux + j][n + i * y_nodes] = dy[f][n] * y_nodes / (x_nodes * frame_mux)
__global__ void k_binary_to_real_backward(const float *__restrict__ dy, float *dx, int node_mux, int frame_mux, int y_nodes, long long xs,
                                          int y_frames, long long ys)
{
    const long long xf = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int xn = blockIdx.y;
    if (xf >= (long long)y_frames * frame_mux) return;
    const float gain = (float)y_nodes / ((float)(y_nodes * node_mux) * (float)frame_mux);
    float g = dy[(size_t)(xn % y_nodes) * ys + xf / frame_mux];
    g *= gain;
    dx[(size_t)xn * xs + xf] = g;
}

}   // namespace bb200

using namespace bb200;

extern "C" int bbcu_bit_fp32_RealToBinary_Forward(const float *x, int *y, const float *dev_thresholds, int threshold_frame_stride,
                                                  unsigned depth_modulation_size, unsigned frame_modulation_size, float input_range_lo,
                                                  float input_range_hi, unsigned point_size, unsigned x_depth_size, unsigned x_frame_size,
                                                  unsigned x_frame_stride, unsigned y_frame_stride, bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(x); BB200_REQUIRE_PTR(y);
    BB200_REQUIRE(depth_modulation_size > 0 && frame_modulation_size > 0 && point_size > 0 && input_range_hi != input_range_lo, BBCU_ERR_BAD_SIZE);
    const unsigned long long out_frames = (unsigned long long)x_frame_size * frame_modulation_size;
    const unsigned long long out_nodes = (unsigned long long)x_depth_size * depth_modulation_size * point_size;
    BB200_REQUIRE(out_frames < (1ull << 31) && out_nodes <= 65535ull * 64, BBCU_ERR_TOO_LARGE);
    BB200_REQUIRE(x_frame_stride >= x_frame_size && (unsigned long long)y_frame_stride * 32 >= out_frames, BBCU_ERR_BAD_STRIDE);
    BB200_REQUIRE(dev_thresholds == nullptr || (unsigned long long)threshold_frame_stride >= out_frames, BBCU_ERR_BAD_STRIDE);
    if (out_frames == 0 || out_nodes == 0) return BBCU_OK;
    BB200_REQUIRE(out_nodes <= 65535, BBCU_ERR_TOO_LARGE);
    k_real_to_binary_bit<<<dim3((unsigned)((out_frames + 255) / 256), (unsigned)out_nodes), 256, 0, as_stream(stream)>>>(
        x, reinterpret_cast<uint32_t *>(y), dev_thresholds, depth_modulation_size, frame_modulation_size, input_range_lo, input_range_hi, point_size,
        x_frame_size, x_frame_stride, y_frame_stride, threshold_frame_stride, (unsigned)out_nodes);
    return launch_status();
}

static int b2r_check(const void *x, const void *y, int node_mux, int frame_mux, int y_nodes, int x_stride, int y_frames, int y_stride, bool xbit)
{
    BB200_REQUIRE_PTR(x); BB200_REQUIRE_PTR(y);
    BB200_REQUIRE(node_mux > 0 && frame_mux > 0 && y_nodes > 0 && y_nodes <= 65535 && y_frames >= 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE((long long)y_nodes * node_mux <= 65535, BBCU_ERR_TOO_LARGE);
    BB200_REQUIRE(y_stride >= y_frames && (long long)x_stride * (xbit ? 32 : 1) >= (long long)y_frames * frame_mux, BBCU_ERR_BAD_STRIDE);
    return BBCU_OK;
}

extern "C" int bbcu_bit_fp32_BinaryToReal_Forward(const int *x, float *y, int node_mux_size, int frame_mux_size, int y_node_size,
                                                  int x_frame_stride, int y_frame_size, int y_frame_stride, bbcu_stream_t stream)
{
    int rc = b2r_check(x, y, node_mux_size, frame_mux_size, y_node_size, x_frame_stride, y_frame_size, y_frame_stride, true);
    if (rc || y_frame_size == 0) return rc;
    k_binary_to_real_forward<true><<<dim3((y_frame_size + 127) / 128, y_node_size), 128, 0, as_stream(stream)>>>(
        x, y, node_mux_size, frame_mux_size, y_node_size, x_frame_stride, y_frame_size, y_frame_stride);
    return launch_status();
}

extern "C" int bbcu_fp32_BinaryToReal_Forward(const float *x, float *y, int node_mux_size, int frame_mux_size, int y_node_size,
                                              int x_frame_stride, int y_frame_size, int y_frame_stride, bbcu_stream_t stream)
{
    int rc = b2r_check(x, y, node_mux_size, frame_mux_size, y_node_size, x_frame_stride, y_frame_size, y_frame_stride, false);
    if (rc || y_frame_size == 0) return rc;
    k_binary_to_real_forward<false><<<dim3((y_frame_size + 127) / 128, y_node_size), 128, 0, as_stream(stream)>>>(
        x, y, node_mux_size, frame_mux_size, y_node_size, x_frame_stride, y_frame_size, y_frame_stride);
    return launch_status();
}

extern "C" int bbcu_fp32_BinaryToReal_Backward(const float *dy, float *dx, int node_mux_size, int frame_mux_size, int y_node_size,
                                               int x_frame_stride, int y_frame_size, int y_frame_stride, bbcu_stream_t stream)
{
    int rc = b2r_check(dy, dx, node_mux_size, frame_mux_size, y_node_size, x_frame_stride, y_frame_size, y_frame_stride, false);
    if (rc || y_frame_size == 0) return rc;
    const long long xf = (long long)y_frame_size * frame_mux_size;
    k_binary_to_real_backward<<<dim3((unsigned)((xf + 255) / 256), y_node_size * node_mux_size), 256, 0, as_stream(stream)>>>(
        dy, dx, node_mux_size, frame_mux_size, y_node_size, x_frame_stride, y_frame_size, y_frame_stride);
    return launch_status();
}
