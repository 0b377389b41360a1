// Neighbours of the LUT path in a training step: the two losses the reference's LUT samples use and the node-group mean
// (bb::Reduce) that maps the last LUT layer to class scores.  Tiny next to the LUT layers (10 class rows against
// thousands of LUT rows); they exist so that a whole step -- forward, loss, backward, Adam -- stays on the device.
//
// Semantics follow the reference's CPU branches:
//   LossSoftmaxCrossEntropy  include/bb/LossSoftmaxCrossEntropy.h:151-205   (operator: include/bbcu/bbcu.h:1507-1519)
//   LossMeanSquaredError     include/bb/LossMeanSquaredError.h:153-172      (operator: include/bbcu/bbcu.h:1487-1500)
//   Reduce                   include/bb/Reduce.h:200-220, 250-268           (no CUDA counterpart in the reference)
#include "common.cuh"

namespace bb200 {

// one thread per (frame, pixel): softmax over the ch_size channel rows node = ch * pix_size + pix
__global__ void k_softmax_cross_entropy(const float *__restrict__ y, const float *__restrict__ t, float *dy, double *loss_buf, float t_sum,
                                        int pix_size, int ch_size, int F, long long stride)
{
    const int f = blockIdx.x * blockDim.x + threadIdx.x;
    if (f >= F) return;
    const float eps = 1.0e-7f;
    double loss = 0.0;
    for (int pix = 0; pix < pix_size; ++pix) {
        float c = -3.402823466e+38f;
        for (int ch = 0; ch < ch_size; ++ch) c = fmaxf(c, y[(size_t)(ch * pix_size + pix) * stride + f]);
        float y_sum = 0.0f, t_max = 0.0f;
        for (int ch = 0; ch < ch_size; ++ch) {
            const size_t o = (size_t)(ch * pix_size + pix) * stride + f;
            y_sum += expf(y[o] - c);
            t_max += t[o];                       // one-hot targets: the sum is the frame's weight
        }
        if (y_sum <= eps) y_sum = eps;
        for (int ch = 0; ch < ch_size; ++ch) {
            const size_t o = (size_t)(ch * pix_size + pix) * stride + f;
            const float softmax = expf(y[o] - c) / y_sum;
            const float tv = t[o];
            if (tv > 0.0f) loss += (double)(logf(softmax + eps) * t_max);
            dy[o] = (t_max * softmax - tv) / t_sum;
        }
    }
    loss_buf[f] = loss;
}

// dy = grad_reduction * (y - t);  loss_buf[block % loss_buf_size] += sum (y - t)^2 * loss_reduction  (NaN terms skipped)
__global__ void __launch_bounds__(256)
k_mean_squared_error(const float *__restrict__ y, const float *__restrict__ t, float *dy, double *loss_buf, int loss_buf_size, int F,
                     long long stride, float grad_reduction, double loss_reduction, int chunks)
{
    __shared__ double red[8];
    const int node = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    const size_t row = (size_t)node * stride;
    const int f0 = chunk * 8192, f1 = min(F, f0 + 8192);
    double acc = 0.0;
    for (int f = f0 + threadIdx.x; f < f1; f += 256) {
        const float g = y[row + f] - t[row + f];
        dy[row + f] = g * grad_reduction;
        const float e = g * g;
        if (e == e) acc += (double)e;
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double s = 0.0;
        for (int w = 0; w < 8; ++w) s += red[w];
        atomicAdd(loss_buf + (blockIdx.x % loss_buf_size), s * loss_reduction);
    }
}

// y[o] = mean_i x[out_nodes * i + o]    /    dx[out_nodes * i + o] = dy[o] / mux
__global__ void k_reduce_forward(const float *__restrict__ x, float *y, int out_nodes, int mux, int F, long long xs, long long ys)
{
    const int f = blockIdx.x * blockDim.x + threadIdx.x;
    const int o = blockIdx.y;
    if (f >= F) return;
    float sum = 0.0f;
    for (int i = 0; i < mux; ++i) sum += x[(size_t)(out_nodes * i + o) * xs + f];
    y[(size_t)o * ys + f] = sum / (float)mux;
}

__global__ void k_reduce_backward(const float *__restrict__ dy, float *dx, int out_nodes, int mux, int F, long long dys, long long dxs)
{
    const int f = blockIdx.x * blockDim.x + threadIdx.x;
    const int o = blockIdx.y;
    if (f >= F) return;
    const float g = dy[(size_t)o * dys + f] / (float)mux;
    for (int i = 0; i < mux; ++i) dx[(size_t)(out_nodes * i + o) * dxs + f] = g;
}

}   // namespace bb200

using namespace bb200;

extern "C" int bbcu_fp32_LossSoftmaxCrossEntropy(const float *y, const float *t, float *dy, double *loss_buf, float t_sum, int pix_size,
                                                 int ch_size, int frame_size, int frame_stride, bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(y); BB200_REQUIRE_PTR(t); BB200_REQUIRE_PTR(dy); BB200_REQUIRE_PTR(loss_buf);
    BB200_REQUIRE(pix_size > 0 && ch_size > 0 && frame_size >= 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE(frame_stride >= frame_size, BBCU_ERR_BAD_STRIDE);
    if (frame_size == 0) return BBCU_OK;
    k_softmax_cross_entropy<<<(frame_size + 127) / 128, 128, 0, as_stream(stream)>>>(y, t, dy, loss_buf, t_sum, pix_size, ch_size, frame_size,
                                                                                   frame_stride);
    return launch_status();
}

extern "C" int bbcu_fp32_LossMeanSquaredError(const float *y, const float *t, float *dy, double *loss_buf, int loss_buf_size, int node_size,
                                              int frame_size, int frame_stride, float grad_reduction, double loss_reduction,
                                              bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(y); BB200_REQUIRE_PTR(t); BB200_REQUIRE_PTR(dy); BB200_REQUIRE_PTR(loss_buf);
    BB200_REQUIRE(loss_buf_size > 0 && node_size >= 0 && frame_size >= 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE(frame_stride >= frame_size, BBCU_ERR_BAD_STRIDE);
    if (node_size == 0 || frame_size == 0) return BBCU_OK;
    const int chunks = (frame_size + 8191) / 8192;
    BB200_REQUIRE((long long)node_size * chunks < (1LL << 31), BBCU_ERR_TOO_LARGE);
    k_mean_squared_error<<<node_size * chunks, 256, 0, as_stream(stream)>>>(y, t, dy, loss_buf, loss_buf_size, frame_size, frame_stride,
                                                                          grad_reduction, loss_reduction, chunks);
    return launch_status();
}

extern "C" int bbcu_fp32_Reduce_Forward(const float *x, float *y, int input_node_size, int output_node_size, int frame_size,
                                        int x_frame_stride, int y_frame_stride, bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(x); BB200_REQUIRE_PTR(y);
    BB200_REQUIRE(output_node_size > 0 && input_node_size >= output_node_size && input_node_size % output_node_size == 0 && frame_size >= 0 &&
                  output_node_size <= 65535, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE(x_frame_stride >= frame_size && y_frame_stride >= frame_size, BBCU_ERR_BAD_STRIDE);
    if (frame_size == 0) return BBCU_OK;
    k_reduce_forward<<<dim3((frame_size + 255) / 256, output_node_size), 256, 0, as_stream(stream)>>>(
        x, y, output_node_size, input_node_size / output_node_size, frame_size, x_frame_stride, y_frame_stride);
    return launch_status();
}

extern "C" int bbcu_fp32_Reduce_Backward(const float *dy, float *dx, int input_node_size, int output_node_size, int frame_size,
                                         int dy_frame_stride, int dx_frame_stride, bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(dy); BB200_REQUIRE_PTR(dx);
    BB200_REQUIRE(output_node_size > 0 && input_node_size >= output_node_size && input_node_size % output_node_size == 0 && frame_size >= 0 &&
                  output_node_size <= 65535, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE(dy_frame_stride >= frame_size && dx_frame_stride >= frame_size, BBCU_ERR_BAD_STRIDE);
    if (frame_size == 0) return BBCU_OK;
    k_reduce_backward<<<dim3((frame_size + 255) / 256, output_node_size), 256, 0, as_stream(stream)>>>(
        dy, dx, output_node_size, input_node_size / output_node_size, frame_size, dy_frame_stride, dx_frame_stride);
    return launch_status();
}
