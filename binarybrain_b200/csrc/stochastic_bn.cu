// Stand-alone StochasticBatchNormalization (scalar gamma/beta batch norm over the frame axis of each node),
// plus the small element-wise operators the LUT layers' callers run every step (W clamp, fill, Adam).
//
// Results follow the reference's CPU branch of that class (include/bb/StochasticBatchNormalization.h:521-617,
// :655-682, :808-852): var = max(0, E[(x-mean)^2]), rstd = 1/(sqrt(var)+1e-7) -- not the old CUDA kernel's
// max(1e-5, .) / rsqrt (cuda/StochasticBatchNormalization.cu:76-96).  Sums over frames are taken in fp64, so
// E[x^2] - mean^2 loses nothing against the CPU's two-pass form.
//
// All four operators are HBM-bound streams over [node][frame] rows: one CTA per (node, 8192-frame chunk),
// 128-bit accesses when the rows are 16-byte aligned.
#include "common.cuh"

namespace bb200 {

constexpr int kChunk = 8192;

__device__ __forceinline__ double block_sum(double v, double *smem)
{
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    v = (threadIdx.x < (blockDim.x >> 5)) ? smem[threadIdx.x] : 0.0;
    if (warp == 0) {
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    }
    return v;   // valid in thread 0
}

template <typename Fn>
__device__ __forceinline__ void for_each_frame(int f0, int f1, bool vec, Fn fn)
{
    if (vec) {
        int f = f0 + threadIdx.x * 4;
        for (; f + 3 < f1; f += blockDim.x * 4) fn(f, 4);
        if (f < f1) fn(f, f1 - f);
    } else {
        for (int f = f0 + threadIdx.x; f < f1; f += blockDim.x) fn(f, 1);
    }
}

// sums[node] += (sum x, sum x^2) over the chunk
__global__ void __launch_bounds__(256)
k_sbn_stats(const float *__restrict__ x, double *sums, int F, long long xs, int chunks)
{
    __shared__ double red[8];
    const int node = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    const float *row = x + (size_t)node * xs;
    const int f0 = chunk * kChunk, f1 = min(F, f0 + kChunk);
    const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
    double s1 = 0.0, s2 = 0.0;
    for_each_frame(f0, f1, vec, [&](int f, int n) {
        if (n == 4) {
            float4 v = __ldg(reinterpret_cast<const float4 *>(row + f));
            s1 += (double)v.x + (double)v.y + (double)v.z + (double)v.w;
            s2 += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
        } else {
            for (int i = 0; i < n; ++i) { float v = __ldg(row + f + i); s1 += v; s2 += (double)v * v; }
        }
    });
    s1 = block_sum(s1, red);
    s2 = block_sum(s2, red);
    if (threadIdx.x == 0) { atomicAdd(sums + 2 * (size_t)node, s1); atomicAdd(sums + 2 * (size_t)node + 1, s2); }
}

__global__ void k_sbn_finalize(const double *__restrict__ sums, float *mean_out, float *rstd_out, float *running_mean, float *running_var,
                               float momentum, int O, int F)
{
    int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= O) return;
    const double m = sums[2 * (size_t)n] / (double)F;
    double v = sums[2 * (size_t)n + 1] / (double)F - m * m;
    const float mean = (float)m;
    const float var  = fmaxf(0.0f, (float)v);
    const float rstd = 1.0f / (sqrtf(var) + 1.0e-7f);
    running_mean[n] = running_mean[n] * momentum + mean * (1.0f - momentum);
    running_var[n]  = running_var[n]  * momentum + var  * (1.0f - momentum);
    mean_out[n] = mean;
    rstd_out[n] = rstd;
}

// mode 0: y = (x - mean) * rstd * gamma + beta      (training / re-forward; b = rstd)
// mode 1: y = gain * x + offset with gain = gamma / (sqrt(var) + 1e-7)   (inference; b = variance)
__global__ void __launch_bounds__(256)
k_sbn_apply(const float *__restrict__ x, float *y, const float *__restrict__ a_buf, const float *__restrict__ b_buf,
            float gamma, float beta, int F, long long xs, int chunks, int mode)
{
    const int node = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    const float *row = x + (size_t)node * xs;
    float *out = y + (size_t)node * xs;
    const int f0 = chunk * kChunk, f1 = min(F, f0 + kChunk);
    const bool vec = ((reinterpret_cast<uintptr_t>(row) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const float mean = a_buf[node];
    float rstd = b_buf[node], gain = 0.0f, offset = 0.0f;
    if (mode == 1) {
        const float sd = sqrtf(rstd) + 1.0e-7f;
        gain = gamma / sd;
        offset = beta - (gamma * mean / sd);
    }
    auto f1x = [&](float v) {
        if (mode == 1) return gain * v + offset;
        float t = (v - mean) * rstd;
        return t * gamma + beta;
    };
    for_each_frame(f0, f1, vec, [&](int f, int n) {
        if (n == 4) {
            float4 v = __ldg(reinterpret_cast<const float4 *>(row + f));
            *reinterpret_cast<float4 *>(out + f) = make_float4(f1x(v.x), f1x(v.y), f1x(v.z), f1x(v.w));
        } else {
            for (int i = 0; i < n; ++i) out[f + i] = f1x(__ldg(row + f + i));
        }
    });
}

// sums[node] += (dstd, dmeanx) with dxn = gamma*dy:  dstd = sum -(dxn*(x-mean)*rstd^2),  dmeanx = sum -(dxn*rstd)
__global__ void __launch_bounds__(256)
k_sbn_backward_stats(const float *__restrict__ x, const float *__restrict__ dy, const float *__restrict__ mean_buf,
                     const float *__restrict__ rstd_buf, double *sums, float gamma, int F, long long xs, long long dys, int chunks)
{
    __shared__ double red[8];
    const int node = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    const float *xr = x + (size_t)node * xs;
    const float *gr = dy + (size_t)node * dys;
    const int f0 = chunk * kChunk, f1 = min(F, f0 + kChunk);
    const bool vec = ((reinterpret_cast<uintptr_t>(xr) | reinterpret_cast<uintptr_t>(gr)) & 15) == 0;
    const float mean = mean_buf[node], rstd = rstd_buf[node], rstd2 = rstd * rstd;
    double dstd = 0.0, dmeanx = 0.0;
    auto one = [&](float xv, float g) {
        float dxn = gamma * g;
        dstd   -= (double)(dxn * (xv - mean) * rstd2);
        dmeanx -= (double)(dxn * rstd);
    };
    for_each_frame(f0, f1, vec, [&](int f, int n) {
        if (n == 4) {
            float4 a = __ldg(reinterpret_cast<const float4 *>(xr + f));
            float4 g = __ldg(reinterpret_cast<const float4 *>(gr + f));
            one(a.x, g.x); one(a.y, g.y); one(a.z, g.z); one(a.w, g.w);
        } else {
            for (int i = 0; i < n; ++i) one(__ldg(xr + f + i), __ldg(gr + f + i));
        }
    });
    dstd = block_sum(dstd, red);
    dmeanx = block_sum(dmeanx, red);
    if (threadIdx.x == 0) { atomicAdd(sums + 2 * (size_t)node, dstd); atomicAdd(sums + 2 * (size_t)node + 1, dmeanx); }
}

__global__ void __launch_bounds__(256)
k_sbn_backward_apply(const float *__restrict__ x, const float *__restrict__ dy, float *dx, const float *__restrict__ mean_buf,
                     const float *__restrict__ rstd_buf, const double *__restrict__ sums, float gamma, float rF, int F,
                     long long xs, long long dys, int chunks)
{
    const int node = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    const float *xr = x + (size_t)node * xs;
    const float *gr = dy + (size_t)node * dys;
    float *out = dx + (size_t)node * dys;
    const int f0 = chunk * kChunk, f1 = min(F, f0 + kChunk);
    const bool vec = ((reinterpret_cast<uintptr_t>(xr) | reinterpret_cast<uintptr_t>(gr) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const float mean = mean_buf[node], rstd = rstd_buf[node];
    const float dvar  = (float)sums[2 * (size_t)node] * rstd;
    const float dmean = ((float)sums[2 * (size_t)node + 1] - (mean * dvar)) * rF;
    auto one = [&](float xv, float g) {
        float dxc = (g * gamma) * rstd;
        return dxc + dmean + (xv * dvar * rF);
    };
    for_each_frame(f0, f1, vec, [&](int f, int n) {
        if (n == 4) {
            float4 a = __ldg(reinterpret_cast<const float4 *>(xr + f));
            float4 g = __ldg(reinterpret_cast<const float4 *>(gr + f));
            *reinterpret_cast<float4 *>(out + f) = make_float4(one(a.x, g.x), one(a.y, g.y), one(a.z, g.z), one(a.w, g.w));
        } else {
            for (int i = 0; i < n; ++i) out[f + i] = one(__ldg(xr + f + i), __ldg(gr + f + i));
        }
    });
}

// ------------------------------------------------------------------------------------------- element-wise
__global__ void k_clamp(float *dst, const float *__restrict__ src, float lo, float hi, int n)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) dst[i] = fmaxf(lo, fminf(hi, src[i]));
}

__global__ void k_set(float *dst, float a, int n)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) dst[i] = a;
}

// One grid row per tensor of the table (the reference: one block per tensor, cuda/OptimizerAdam.cu:12-48).
__global__ void k_adam(const int *__restrict__ size_table, float *const *params, float *const *grads, float *const *m_tab, float *const *v_tab,
                       float lr_t, float beta1, float beta2)
{
    const int t = blockIdx.y;
    const int n = size_table[t];
    float *p = params[t], *m = m_tab[t], *v = v_tab[t];
    const float *g = grads[t];
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float gi = g[i], mi = m[i], vi = v[i];
        mi += (1.0f - beta1) * (gi - mi);
        vi += (1.0f - beta2) * (gi * gi - vi);
        p[i] -= lr_t * mi / (sqrtf(vi) + 1.0e-7f);
        m[i] = mi;
        v[i] = vi;
    }
}

static int sbn_check(const void *x, const void *y, int O, int F, int stride)
{
    BB200_REQUIRE_PTR(x); BB200_REQUIRE_PTR(y);
    BB200_REQUIRE(O >= 0 && F >= 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE(stride >= F, BBCU_ERR_BAD_STRIDE);
    BB200_REQUIRE((long long)O * ((F + kChunk - 1) / kChunk) < (1LL << 31), BBCU_ERR_TOO_LARGE);
    return BBCU_OK;
}

}   // namespace bb200

using namespace bb200;

extern "C" int bbcu_fp32_StochasticBatchNormalization_ForwardTraining(const float *x, float *y, float *mean, float *rstd, float *rmean,
                                                                      float *rvar, float gamma, float beta, float momentum, int node_size,
                                                                      int frame_size, int frame_stride, bbcu_stream_t stream)
{
    int rc = sbn_check(x, y, node_size, frame_size, frame_stride);
    if (rc) return rc;
    BB200_REQUIRE_PTR(mean); BB200_REQUIRE_PTR(rstd); BB200_REQUIRE_PTR(rmean); BB200_REQUIRE_PTR(rvar);
    BB200_REQUIRE(frame_size > 0 || node_size == 0, BBCU_ERR_BAD_SIZE);
    if (node_size == 0) return BBCU_OK;
    cudaStream_t st = as_stream(stream);
    double *sums = static_cast<double *>(stream_scratch(st, sizeof(double) * 2 * (size_t)node_size));
    BB200_REQUIRE(sums != nullptr, BBCU_ERR_NO_MEMORY);
    BB200_CUDA(cudaMemsetAsync(sums, 0, sizeof(double) * 2 * (size_t)node_size, st));
    const int chunks = (frame_size + kChunk - 1) / kChunk;
    k_sbn_stats<<<node_size * chunks, 256, 0, st>>>(x, sums, frame_size, frame_stride, chunks);
    BB200_CUDA(cudaPeekAtLastError());
    k_sbn_finalize<<<(node_size + 255) / 256, 256, 0, st>>>(sums, mean, rstd, rmean, rvar, momentum, node_size, frame_size);
    BB200_CUDA(cudaPeekAtLastError());
    k_sbn_apply<<<node_size * chunks, 256, 0, st>>>(x, y, mean, rstd, gamma, beta, frame_size, frame_stride, chunks, 0);
    return launch_status();
}

extern "C" int bbcu_fp32_StochasticBatchNormalization_ReForward(const float *x, float *y, const float *mean, const float *rstd, float gamma,
                                                                float beta, int node_size, int frame_size, int frame_stride,
                                                                bbcu_stream_t stream)
{
    int rc = sbn_check(x, y, node_size, frame_size, frame_stride);
    if (rc) return rc;
    BB200_REQUIRE_PTR(mean); BB200_REQUIRE_PTR(rstd);
    if (node_size == 0 || frame_size == 0) return BBCU_OK;
    const int chunks = (frame_size + kChunk - 1) / kChunk;
    k_sbn_apply<<<node_size * chunks, 256, 0, as_stream(stream)>>>(x, y, mean, rstd, gamma, beta, frame_size, frame_stride, chunks, 0);
    return launch_status();
}

extern "C" int bbcu_fp32_StochasticBatchNormalization_ForwardInference(const float *x, float *y, const float *rmean, const float *rvar,
                                                                       float gamma, float beta, int node_size, int frame_size,
                                                                       int frame_stride, bbcu_stream_t stream)
{
    int rc = sbn_check(x, y, node_size, frame_size, frame_stride);
    if (rc) return rc;
    BB200_REQUIRE_PTR(rmean); BB200_REQUIRE_PTR(rvar);
    if (node_size == 0 || frame_size == 0) return BBCU_OK;
    const int chunks = (frame_size + kChunk - 1) / kChunk;
    k_sbn_apply<<<node_size * chunks, 256, 0, as_stream(stream)>>>(x, y, rmean, rvar, gamma, beta, frame_size, frame_stride, chunks, 1);
    return launch_status();
}

extern "C" int bbcu_fp32_StochasticBatchNormalization_Backward(const float *x, const float *dy, float *dx, const float *mean, const float *rstd,
                                                               float gamma, float reciprocal_frame_size, int node_size, int frame_size,
                                                               int frame_stride, int x_frame_stride, bbcu_stream_t stream)
{
    int rc = sbn_check(x, dx, node_size, frame_size, frame_stride);
    if (rc) return rc;
    BB200_REQUIRE_PTR(dy); BB200_REQUIRE_PTR(mean); BB200_REQUIRE_PTR(rstd);
    BB200_REQUIRE(x_frame_stride >= frame_size, BBCU_ERR_BAD_STRIDE);
    if (node_size == 0 || frame_size == 0) return BBCU_OK;
    cudaStream_t st = as_stream(stream);
    double *sums = static_cast<double *>(stream_scratch(st, sizeof(double) * 2 * (size_t)node_size));
    BB200_REQUIRE(sums != nullptr, BBCU_ERR_NO_MEMORY);
    BB200_CUDA(cudaMemsetAsync(sums, 0, sizeof(double) * 2 * (size_t)node_size, st));
    const int chunks = (frame_size + kChunk - 1) / kChunk;
    k_sbn_backward_stats<<<node_size * chunks, 256, 0, st>>>(x, dy, mean, rstd, sums, gamma, frame_size, x_frame_stride, frame_stride, chunks);
    BB200_CUDA(cudaPeekAtLastError());
    k_sbn_backward_apply<<<node_size * chunks, 256, 0, st>>>(x, dy, dx, mean, rstd, sums, gamma, reciprocal_frame_size, frame_size,
                                                           x_frame_stride, frame_stride, chunks);
    return launch_status();
}

extern "C" int bbcu_fp32_Vector_clamp(float *dst, const float *src, float lo, float hi, int size, bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(dst); BB200_REQUIRE_PTR(src);
    BB200_REQUIRE(size >= 0, BBCU_ERR_BAD_SIZE);
    if (size == 0) return BBCU_OK;
    int blocks = (size + 255) / 256; if (blocks > 4096) blocks = 4096;
    k_clamp<<<blocks, 256, 0, as_stream(stream)>>>(dst, src, lo, hi, size);
    return launch_status();
}

extern "C" int bbcu_fp32_Vector_set(float *dst, float a, int size, bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(dst);
    BB200_REQUIRE(size >= 0, BBCU_ERR_BAD_SIZE);
    if (size == 0) return BBCU_OK;
    int blocks = (size + 255) / 256; if (blocks > 4096) blocks = 4096;
    k_set<<<blocks, 256, 0, as_stream(stream)>>>(dst, a, size);
    return launch_status();
}

extern "C" int bbcu_fp32_OptimizerAdam(int size, const int *size_table, float *const *params, float *const *grads, float *const *m_tab,
                                       float *const *v_tab, float lr_t, float beta1, float beta2, bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(size_table); BB200_REQUIRE_PTR(params); BB200_REQUIRE_PTR(grads); BB200_REQUIRE_PTR(m_tab); BB200_REQUIRE_PTR(v_tab);
    BB200_REQUIRE(size >= 0 && size <= 65535, BBCU_ERR_BAD_SIZE);
    if (size == 0) return BBCU_OK;
    k_adam<<<dim3(296, size), 256, 0, as_stream(stream)>>>(size_table, params, grads, m_tab, v_tab, lr_t, beta1, beta2);
    return launch_status();
}
