// Host-side helpers shared by the operator launchers: argument checks, launch-error capture,
// per-stream scratch memory and the frame-tile heuristic.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

#include "../../include/bbcu_b200.h"

namespace bb200 {

#define BB200_REQUIRE_PTR(p)   do { if ((p) == nullptr) return BBCU_ERR_NULL_POINTER; } while (0)
#define BB200_REQUIRE(cond, e) do { if (!(cond)) return (e); } while (0)
#define BB200_CUDA(call)       do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { cudaGetLastError(); return (int)e_; } } while (0)

constexpr int kFramesPerIterHost = 128;   // frames one warp covers per iteration (32 lanes x 4)

// Status of the launches just made: a launch error is reported once and cleared, so it cannot resurface in a later call.
inline int launch_status() { return (int)cudaGetLastError(); }

// Device properties read once per device.
struct DeviceInfo {
    int sm_count;
    size_t l2_bytes;
    size_t total_bytes;          // device memory
};
const DeviceInfo &device_info();

// Scratch memory private to (device, stream): grows on demand through the device heap, is reused by
// later calls on the same stream and is released by bbcu_LocalHeap_GarbageCollect().  Stream order
// makes back-to-back calls on one stream safe; different streams get different blocks.  A stream has
// kScratchSlots independent blocks, for callers whose scratch is alive at the same time (slot 0: batch-norm
// sums, slot 1: per-node coefficient / pattern tables of the LUT operators, slot 2: the piece table of the bit Im2Col).
constexpr int kScratchSlots = 3;
void *stream_scratch(cudaStream_t stream, size_t bytes, int slot = 0);

// Pass 1 of the DifferentiableLut6 training forward (raw LUT values into y, fp64 sums per node); with may_allocate = false
// it takes nothing from the heap or the stream scratch.
int dl6_forward_stats(const float *x, float *y, const int *idx, const float *W, double *dev_sums, float unbinarize_bias, int node_size,
                      int frame_size, int frame_stride, int lut_binarize, int binary_mode, bool may_allocate, cudaStream_t st);

// Frames handled by one CTA pass.  The gathered input rows of a frame tile (and, in the backward
// pass, the dx rows it reduces into) have to stay resident in L2 while every output node of the
// layer consumes them, so the tile narrows as the layer widens; it widens again, up to max_tile,
// while that still leaves enough CTAs to fill the machine.
int frame_tile(long long rows_touched, int bits_per_row_frame, int node_groups, int frame_size, int max_tile);

// Bit-in / bit-out LUT layers evaluated through a per-node pattern table and the BinaryLut6 kernel (binary_mode.cu).  Both return
// BBCU_ERR_NO_MEMORY when their scratch cannot be had, in which case the caller runs the per-frame kernels instead.
int bit_forward_by_table(bool with_bn, const int *x, int *y, const int *idx, const float *W, const float *rmean, const float *rvar, float gamma,
                         float beta, float bias, int O, int F, int stride, int lut_binarize, cudaStream_t st);
int dl6_bit_forward_training_by_table(const int *x, int *y, const int *idx, const float *W, float *mean, float *rstd, float *rmean, float *rvar,
                                      float gamma, float beta, float momentum, float bias, int O, int F, int stride, int lut_binarize,
                                      cudaStream_t st);

int bit_fp32_forward_by_table(const int *x, float *y, const int *idx, const float *W, float bias, int O, int F, long long xs, long long ys,
                              int lut_binarize, cudaStream_t st);

int bit_backward_by_table(bool bn, bool x_is_fp32, const void *x, const float *dy, float *dx, const int *idx, const float *W, float *dW,
                          const float *mean, const float *rstd, float *dmean_out, float *dvar_out, float gamma, float beta, float bias, int O, int F,
                          long long xs, long long fs, int lut_binarize, cudaStream_t st);

// The batch-norm backward of a binary-mode layer in two halves for frame-sharded callers (the caller adds `sums` over the ranks in
// between); both decline with BBCU_ERR_NO_MEMORY like the calls above.
int bit_backward_stats_by_table(bool x_is_fp32, const void *x, const float *dy, const int *idx, const float *W, const float *mean, const float *rstd,
                                double *sums, float gamma, float beta, float bias, int O, int F, long long xs, long long fs, int lut_binarize,
                                cudaStream_t st);
int bit_backward_apply_by_table(bool x_is_fp32, const void *x, const float *dy, float *dx, const int *idx, const float *W, float *dW, const float *mean,
                                const float *rstd, const double *sums, float *dmean_out, float *dvar_out, float gamma, float beta, float bias, int O,
                                int F, long long xs, long long fs, long long total_frames, int lut_binarize, cudaStream_t st);

int f32_binary_forward_by_table(int mode, const float *x, float *y, const int *idx, const float *W, float *mean, float *rstd, float *rmean,
                                float *rvar, float gamma, float beta, float momentum, float bias, int O, int F, long long fs, int lut_binarize,
                                cudaStream_t st);

// Per-device int in the library's device image (zero until a kernel records a fault); nothing is allocated for it.
int *fault_word();

inline cudaStream_t as_stream(bbcu_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

}   // namespace bb200
