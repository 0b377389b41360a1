/* bbcu_b200.h -- C ABI of the sm_100a implementation of BinaryBrain's LUT6 hot path.
 *
 * Every entry point replaces one operator of BinaryBrain's CUDA layer (include/bbcu/bbcu.h in
 * ryuz/BinaryBrain v4.3.2; the citation beside each declaration is the prototype it replaces).
 * The reference declares the LUT operators as C++ templates on the LUT width N; a C symbol cannot
 * be a template, so N = 6 is folded into the name ("...Lut6_..."), the spelling the reference's own
 * raw-kernel harness already uses (tests/cuda/StochasticLut6_Test.cpp:60,174).  Argument order and
 * meaning are the reference's, with these fixed rules:
 *
 *   - every pointer is a DEVICE pointer on the current device unless its name starts with host_;
 *   - fp32 frame buffers are node-major: element (frame f, node n) at buf[n*frame_stride + f];
 *     bit buffers hold 32 frames per 32-bit word, frame f = bit (f & 31) of word n*stride + (f >> 5)
 *     (include/bb/FrameBuffer.h:28-46, include/bb/DataType.h:612-647); strides are in ELEMENTS
 *     (floats or 32-bit words), as the reference's callers pass them;
 *   - input_index is [output_node][6] int32, W is [output_node][64] fp32, bit k of the table index
 *     is input k;
 *   - the last argument is the CUDA stream (a cudaStream_t passed as void*, NULL = default
 *     stream).  All work is enqueued on that stream.  The host is not synchronised, with one exception: a call that has
 *     to grow its per-stream scratch (below) allocates, and waits for the stream before it returns the outgrown block; such
 *     a call -- the first one on a stream, or the first one of a larger layer -- belongs outside of stream capture;
 *   - return value: 0 on success, BBCU_ERR_* (< 0) for a rejected argument, a cudaError_t (> 0)
 *     if the CUDA runtime reported one (reported once, then cleared).  Nothing exits the process (the reference's macros call
 *     exit(1), include/bbcu/bbcu_util.h:17-36);
 *   - scratch: the fp32 backward operators use the caller's dev_dx_tmp when it is given, 16-byte aligned and at least 512 bytes
 *     per output node.  Otherwise, and for the operators whose reference signature carries no scratch, the LUT operators keep
 *     per-stream work areas in the device heap below: per-node sums, coefficient and pattern tables (at most ~1 KiB per output
 *     node) and, for DifferentiableLut6 in binary mode on fp32 frames, one pattern byte per node-frame (node_size *
 *     frame_stride bytes; above 1 GiB the operator runs its scratch-free kernels instead).  The first call on a stream
 *     allocates them, later calls reuse them, and bbcu_LocalHeap_GarbageCollect releases them.
 *     ..._ForwardTraining_NoAlloc is the variant that never allocates.
 *
 * Results follow the reference's CPU branches (the header-only path in include/bb), which is what
 * parity is measured against; where the reference's old CUDA kernels differ from its CPU code the
 * CPU code wins.  dev_reverse_index of the backward operators is accepted for signature compatibility and
 * not read: the input gradients of a node are added to dx with 128-bit floating-point reductions
 * (red.global.add.v4.f32) that L2 resolves, instead of going through a [nodes*6][frames] temporary and a
 * gather by reverse index; dev_dx_tmp serves as plain scratch (see above).
 */
#ifndef BBCU_B200_H
#define BBCU_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *bbcu_stream_t;

#define BBCU_OK                 0
#define BBCU_ERR_NULL_POINTER  (-1)
#define BBCU_ERR_BAD_SIZE      (-2)
#define BBCU_ERR_BAD_STRIDE    (-3)
#define BBCU_ERR_NO_DEVICE     (-4)
#define BBCU_ERR_NO_MEMORY     (-5)
#define BBCU_ERR_TOO_LARGE     (-6)

/* Human-readable text for a return value of any function below. */
const char *bbcu_b200_error_string(int status);
/* ABI version of this library (bumped when a signature changes). */
int bbcu_b200_abi_version(void);
/* Synchronises the current device and returns the first fault code one of this library's kernels recorded since the last call
 * (0 = none, 1 = a bounded wait on an asynchronous copy expired, -1 = the query itself failed).  Kernels never trap or spin
 * forever: a wait that does not complete is abandoned, recorded here, and the kernel returns. */
int bbcu_b200_device_fault(void);
/* Self-test of that path: one warp waits, with a small attempt limit, on a barrier that nothing completes, gives up, records fault
 * code 1 and returns (nothing hangs, nothing faults); bbcu_b200_device_fault() then reports 1 once. */
int bbcu_b200_selftest_wait_expiry(bbcu_stream_t stream);

/* ------------------------------------------------------------------ Manager: include/bbcu/bbcu.h:49-55, cuda/Manager.cu:15-55 */
int  bbcu_GetDeviceCount(void);
int  bbcu_GetDevice(void);
void bbcu_SetDevice(int device);
void bbcu_SetHostOnly(int host_only);
int  bbcu_IsHostOnly(void);
int  bbcu_IsDeviceAvailable(void);

/* ------------------------------------------------------------------ Device heap: include/bbcu/bbcu.h:63-67, cuda/LocalHeap.cu:13-201
 * Caching allocator over cudaMalloc, one pool per device, thread-safe.  Malloc returns NULL when the device is out of
 * memory even after the cache has been released (the reference asserts).  Free only returns the block to the cache. */
void  *bbcu_LocalHeap_Malloc(size_t size);
void   bbcu_LocalHeap_Free(void *ptr);
size_t bbcu_LocalHeap_GetMaxAllocSize(void);
size_t bbcu_LocalHeap_GetAllocatedSize(void);
void   bbcu_LocalHeap_GarbageCollect(void);
/* Additive: artificial cap on live+cached bytes (0 = none), used to exercise the out-of-memory path without exhausting a GPU. */
void   bbcu_LocalHeap_SetByteLimit(size_t bytes);

/* ------------------------------------------------------------------ StochasticLut6: include/bbcu/bbcu.h:667-761 */
/* bbcu_fp32_StochasticLut_Forward<6>, include/bbcu/bbcu.h:667-681.  y = clip(lut(x), 0, 1). */
int bbcu_fp32_StochasticLut6_Forward(const float *dev_x_buf, float *dev_y_buf, const int *dev_input_index, const float *dev_W,
                                     int node_size, int frame_size, int frame_stride,
                                     int input_binary, int lut_binarize, float unbinarize_bias, bbcu_stream_t stream);
/* bbcu_bit_fp32_StochasticLut_Forward<6>, include/bbcu/bbcu.h:683-697.  Bit-packed x, fp32 y. */
int bbcu_bit_fp32_StochasticLut6_Forward(const int *dev_x_buf, float *dev_y_buf, const int *dev_input_index, const float *dev_W,
                                         int node_size, int frame_size, int frame_stride, int bin_frame_stride,
                                         int lut_binarize, float unbinarize_bias, bbcu_stream_t stream);
/* bbcu_bit_bit_fp32_StochasticLut_Forward<6>, include/bbcu/bbcu.h:699-712.  Bit-packed x and y (y = lut(x) > 0.5). */
int bbcu_bit_bit_fp32_StochasticLut6_Forward(const int *dev_x_buf, int *dev_y_buf, const int *dev_input_index, const float *dev_W,
                                             int node_size, int frame_size, int frame_stride,
                                             int lut_binarize, float unbinarize_bias, bbcu_stream_t stream);
/* bbcu_fp32_StochasticLut_Backward<6>, include/bbcu/bbcu.h:715-737.  dx overwritten, dW accumulated into. */
int bbcu_fp32_StochasticLut6_Backward(const float *dev_x_buf, const float *dev_dy_buf, float *dev_dx_buf, float *dev_dx_tmp,
                                      const int *dev_input_index, const int *dev_reverse_index, const float *dev_W, float *dev_dW,
                                      int reverse_index_stride, int input_node_size, int output_node_size,
                                      int frame_size, int frame_stride, int tmp_frame_size, int tmp_frame_stride,
                                      int input_binary, int lut_binarize, float unbinarize_bias, bbcu_stream_t stream);
/* bbcu_bit_fp32_StochasticLut_Backward<6>, include/bbcu/bbcu.h:739-761. */
int bbcu_bit_fp32_StochasticLut6_Backward(const int *dev_x_buf, const float *dev_dy_buf, float *dev_dx_buf, float *dev_dx_tmp,
                                          const int *dev_input_index, const int *dev_reverse_index, const float *dev_W, float *dev_dW,
                                          int reverse_index_stride, int input_node_size, int output_node_size,
                                          int frame_size, int frame_stride, int bin_frame_stride, int tmp_frame_size, int tmp_frame_stride,
                                          int lut_binarize, float unbinarize_bias, bbcu_stream_t stream);

/* ------------------------------------------------------------------ DifferentiableLut6: include/bbcu/bbcu.h:518-660 */
/* bbcu_fp32_DifferentiableLutN_ForwardTraining<6>, include/bbcu/bbcu.h:518-539.
 * Writes y, mean, rstd; updates running_mean / running_var with `momentum`. */
int bbcu_fp32_DifferentiableLut6_ForwardTraining(const float *dev_x_buf, float *dev_y_buf, const int *dev_input_index, const float *dev_W,
                                                 float *dev_mean_buf, float *dev_rstd_buf, float *dev_running_mean_buf, float *dev_running_var_buf,
                                                 float gamma, float beta, float momentum, float unbinarize_bias,
                                                 int node_size, int frame_size, int frame_stride, int lut_binarize, int binary_mode,
                                                 bbcu_stream_t stream);
/* bbcu_bit_fp32_DifferentiableLutN_ForwardTraining<6>, include/bbcu/bbcu.h:541-561.  frame_stride in 32-bit words (x and y). */
int bbcu_bit_fp32_DifferentiableLut6_ForwardTraining(const int *dev_x_buf, int *dev_y_buf, const int *dev_input_index, const float *dev_W,
                                                     float *dev_mean_buf, float *dev_rstd_buf, float *dev_running_mean_buf, float *dev_running_var_buf,
                                                     float gamma, float beta, float momentum, float unbinarize_bias,
                                                     int node_size, int frame_size, int frame_stride, int lut_binarize,
                                                     bbcu_stream_t stream);
/* bbcu_fp32_DifferentiableLutN_ForwardInference<6>, include/bbcu/bbcu.h:563-581. */
int bbcu_fp32_DifferentiableLut6_ForwardInference(const float *dev_x_buf, float *dev_y_buf, const int *dev_input_index, const float *dev_W,
                                                  const float *dev_running_mean_buf, const float *dev_running_var_buf,
                                                  float gamma, float beta, float unbinarize_bias,
                                                  int node_size, int frame_size, int frame_stride, int lut_binarize, int binary_mode,
                                                  bbcu_stream_t stream);
/* bbcu_bit_fp32_DifferentiableLutN_ForwardInference<6>, include/bbcu/bbcu.h:583-600. */
int bbcu_bit_fp32_DifferentiableLut6_ForwardInference(const int *dev_x_buf, int *dev_y_buf, const int *dev_input_index, const float *dev_W,
                                                      const float *dev_running_mean_buf, const float *dev_running_var_buf,
                                                      float gamma, float beta, float unbinarize_bias,
                                                      int node_size, int frame_size, int frame_stride, int lut_binarize,
                                                      bbcu_stream_t stream);
/* bbcu_fp32_DifferentiableLutN_Backward<6>, include/bbcu/bbcu.h:602-630.
 * dev_dmean_tmp / dev_dvar_tmp ([output_node_size] fp32) receive the batch-norm mean / variance gradients. */
int bbcu_fp32_DifferentiableLut6_Backward(const float *dev_x_buf, const float *dev_dy_buf, float *dev_dx_buf, float *dev_dx_tmp,
                                          const int *dev_input_index, const int *dev_reverse_index, const float *dev_W, float *dev_dW,
                                          const float *dev_mean_buf, const float *dev_rstd_buf, float *dev_dmean_tmp, float *dev_dvar_tmp,
                                          float gamma, float beta, float unbinarize_bias,
                                          int reverse_index_stride, int input_node_size, int output_node_size,
                                          int frame_size, int frame_stride, int tmp_frame_size, int tmp_frame_stride,
                                          int lut_binarize, int binary_mode, bbcu_stream_t stream);
/* bbcu_bit_fp32_DifferentiableLutN_Backward<6>, include/bbcu/bbcu.h:632-660.  frame_stride: dy/dx floats; x_frame_stride: x words. */
int bbcu_bit_fp32_DifferentiableLut6_Backward(const int *dev_x_buf, const float *dev_dy_buf, float *dev_dx_buf, float *dev_dx_tmp,
                                              const int *dev_input_index, const int *dev_reverse_index, const float *dev_W, float *dev_dW,
                                              const float *dev_mean_buf, const float *dev_rstd_buf, float *dev_dmean_tmp, float *dev_dvar_tmp,
                                              float gamma, float beta, float unbinarize_bias,
                                              int reverse_index_stride, int input_node_size, int output_node_size,
                                              int frame_size, int frame_stride, int x_frame_stride, int tmp_frame_size, int tmp_frame_stride,
                                              int lut_binarize, bbcu_stream_t stream);

/* ------------------------------------------------------------------ StochasticBatchNormalization: include/bbcu/bbcu.h:883-942 */
int bbcu_fp32_StochasticBatchNormalization_ForwardTraining(const float *dev_x_buf, float *dev_y_buf, float *dev_mean_buf, float *dev_rstd_buf,
                                                           float *dev_running_mean_buf, float *dev_running_var_buf,
                                                           float gamma, float beta, float momentum,
                                                           int node_size, int frame_size, int frame_stride, bbcu_stream_t stream);
int bbcu_fp32_StochasticBatchNormalization_ReForward(const float *dev_x_buf, float *dev_y_buf, const float *dev_mean_buf, const float *dev_rstd_buf,
                                                     float gamma, float beta, int node_size, int frame_size, int frame_stride, bbcu_stream_t stream);
int bbcu_fp32_StochasticBatchNormalization_ForwardInference(const float *dev_x_buf, float *dev_y_buf,
                                                            const float *dev_running_mean_buf, const float *dev_running_var_buf,
                                                            float gamma, float beta, int node_size, int frame_size, int frame_stride, bbcu_stream_t stream);
int bbcu_fp32_StochasticBatchNormalization_Backward(const float *dev_x_buf, const float *dev_dy_buf, float *dev_dx_buf,
                                                    const float *dev_mean_buf, const float *dev_rstd_buf, float gamma, float reciprocal_frame_size,
                                                    int node_size, int frame_size, int frame_stride, int x_frame_stride, bbcu_stream_t stream);

/* ------------------------------------------------------------------ BinaryLut6: include/bbcu/bbcu.h:285-295, cuda/BinaryLut6.cu:165-196
 * dev_table is [node][2] int32: bit i of the 64-bit table is the output for input index i (include/bb/BinaryLutN.h:43-46).
 * Unlike the reference (one block per node in grid.y, cuda/BinaryLut6.cu:179-180) any node_size up to INT_MAX works.
 * The reference spells it "BinatyLut6"; both spellings are exported. */
int bbcu_bit_BinaryLut6_Forward(const int *dev_x_buf, int *dev_y_buf, const int *dev_input_index, const int *dev_table,
                                int node_size, int frame_size, int frame_stride, bbcu_stream_t stream);
int bbcu_bit_BinatyLut6_Forward(const int *dev_x_buf, int *dev_y_buf, const int *dev_input_index, const int *dev_table,
                                int node_size, int frame_size, int frame_stride, bbcu_stream_t stream);

/* Additive: the same operator evaluated with the table bytes as lop3 immediates (15 logic operations per 32 frames instead of 63, one
 * indexed branch per table byte).  Bit-identical results; measured slower than the default on B200 (instruction fetch of the
 * dispatched case bodies) and kept so that the comparison can be re-measured.  Rows must be 16-byte aligned: frame_stride a
 * multiple of 4 words and aligned base pointers, BBCU_ERR_BAD_STRIDE otherwise. */
int bbcu_bit_BinaryLut6_Forward_Lop3Immediate(const int *dev_x_buf, int *dev_y_buf, const int *dev_input_index, const int *dev_table,
                                              int node_size, int frame_size, int frame_stride, bbcu_stream_t stream);

/* Additive: the same operator on HOST frame buffers (what a caller does that keeps its FrameBuffers in host memory,
 * include/bb/Memory.h:524-662).  Uploads x in frame chunks, runs the kernel per chunk and downloads y, with upload, kernel and
 * download of neighbouring chunks overlapped on three internal streams; returns when y is complete.  frame_stride is the HOST row
 * stride in 32-bit words.  Use page-locked buffers (bbcu_b200_host_alloc) for full PCIe overlap.  One such call at a time per process. */
int bbcu_host_bit_BinaryLut6_Forward(const int *host_x_buf, int *host_y_buf, const int *host_input_index, const int *host_table,
                                     int input_node_size, int node_size, int frame_size, int frame_stride);
void *bbcu_b200_host_alloc(size_t bytes);
void  bbcu_b200_host_free(void *ptr);

/* ------------------------------------------------------------------ FrameBuffer helpers (the container either side of the path) */
/* bbcu_int32_FrameBufferCopy, include/bbcu/bbcu.h:265-278 (FrameBuffer::CopyTo, include/bb/FrameBuffer.h:481-535): copies a block of
 * node_size rows x frame_size 32-bit words between two frame buffers; offsets and strides in words (fp32 frames, or 32 bit frames). */
int bbcu_int32_FrameBufferCopy(int *dev_dst_buf, const int *dev_src_buf, int node_size, int dst_node_offset, int src_node_offset,
                               int frame_size, int dst_frame_offset, int src_frame_offset, int dst_frame_stride, int src_frame_stride,
                               bbcu_stream_t stream);
/* bbcu_ConvBitToReal<float>, include/bbcu/bbcu.h:247-258 (FrameBuffer::ConvertTo, include/bb/FrameBuffer.h:843-866): y = bit ? value1 : value0. */
int bbcu_fp32_ConvBitToReal(const int *dev_x_buf, float *dev_y_buf, float value0, float value1, int node_size, int frame_size,
                            int x_frame_stride, int y_frame_stride, bbcu_stream_t stream);

/* ------------------------------------------------------------------ Neighbours of the path that its callers need every step */
/* bbcu_fp32_Vector_clamp, include/bbcu/bbcu.h:191-198 (the W clamp of DifferentiableLutN.h:605-608 / StochasticLutN.h:451). */
int bbcu_fp32_Vector_clamp(float *dev_dst, const float *dev_src, float lo, float hi, int size, bbcu_stream_t stream);
/* bbcu_fp32_Vector_set, include/bbcu/bbcu.h:89-94. */
int bbcu_fp32_Vector_set(float *dev_dst, float a, int size, bbcu_stream_t stream);
/* bbcu_fp32_OptimizerAdam, include/bbcu/bbcu.h:1560-1572, cuda/OptimizerAdam.cu:12-48.  The tables are DEVICE arrays of `size`
 * entries.  m += (1-b1)(g-m); v += (1-b2)(g*g-v); p -= lr_t*m/(sqrt(v)+1e-7).  Gradients are left untouched. */
int bbcu_fp32_OptimizerAdam(int size, const int *dev_size_table, float *const *dev_params_buf_table, float *const *dev_grads_buf_table,
                            float *const *dev_m_buf_table, float *const *dev_v_buf_table, float lr_t, float beta1, float beta2,
                            bbcu_stream_t stream);

/* bbcu_LossSoftmaxCrossEntropy<float>, include/bbcu/bbcu.h:1507-1519: per frame and pixel a softmax over the ch_size channel rows
 * (node = ch * pix_size + pix); dy = (t_weight * softmax - t) / t_sum; dev_loss_buf[frame] = sum log(softmax + 1e-7) * t_weight. */
int bbcu_fp32_LossSoftmaxCrossEntropy(const float *dev_y_buf, const float *dev_t_buf, float *dev_dy_buf, double *dev_loss_buf, float t_sum,
                                      int pix_size, int ch_size, int frame_size, int frame_stride, bbcu_stream_t stream);
/* bbcu_fp32_LossMeanSquaredError, include/bbcu/bbcu.h:1487-1500: dy = grad_reduction * (y - t); the squared errors times loss_reduction
 * are ADDED into dev_loss_buf[0 .. loss_buf_size) (the caller sums the buffer). */
int bbcu_fp32_LossMeanSquaredError(const float *dev_y_buf, const float *dev_t_buf, float *dev_dy_buf, double *dev_loss_buf, int loss_buf_size,
                                   int node_size, int frame_size, int frame_stride, float grad_reduction, double loss_reduction,
                                   bbcu_stream_t stream);
/* Additive (the reference's bb::Reduce has only a CPU branch, include/bb/Reduce.h:200-268): y[o] = mean_i x[output_node_size * i + o]. */
int bbcu_fp32_Reduce_Forward(const float *dev_x_buf, float *dev_y_buf, int input_node_size, int output_node_size, int frame_size,
                             int x_frame_stride, int y_frame_stride, bbcu_stream_t stream);
int bbcu_fp32_Reduce_Backward(const float *dev_dy_buf, float *dev_dx_buf, int input_node_size, int output_node_size, int frame_size,
                              int dy_frame_stride, int dx_frame_stride, bbcu_stream_t stream);

/* bbcu_bit_RealToBinary_Forward<float>, include/bbcu/bbcu.h:1355-1369, with one added argument pair: dev_thresholds == NULL gives the
 * deterministic modulation of the reference's operator (include/bb/RealToBinary.h:309-345, binary mode); otherwise it is an fp32 frame
 * buffer [input node][output frame] (row stride threshold_frame_stride) and bit = modulated x > threshold, the form the reference
 * evaluates on the host with a value generator (:352-398).  Output frames = x_frame_size * frame_modulation_size, bit-packed. */
int bbcu_bit_fp32_RealToBinary_Forward(const float *dev_x_buf, int *dev_y_buf, const float *dev_thresholds, int threshold_frame_stride,
                                       unsigned depth_modulation_size, unsigned frame_modulation_size, float input_range_lo,
                                       float input_range_hi, unsigned point_size, unsigned x_depth_size, unsigned x_frame_size,
                                       unsigned x_frame_stride, unsigned y_frame_stride, bbcu_stream_t stream);
/* bbcu_bit_fp32_BinaryToReal_Forward / bbcu_fp32_BinaryToReal_Forward / bbcu_fp32_BinaryToReal_Backward, include/bbcu/bbcu.h:1376-1413. */
int bbcu_bit_fp32_BinaryToReal_Forward(const int *dev_x_buf, float *dev_y_buf, int node_mux_size, int frame_mux_size, int y_node_size,
                                       int x_frame_stride, int y_frame_size, int y_frame_stride, bbcu_stream_t stream);
int bbcu_fp32_BinaryToReal_Forward(const float *dev_x_buf, float *dev_y_buf, int node_mux_size, int frame_mux_size, int y_node_size,
                                   int x_frame_stride, int y_frame_size, int y_frame_stride, bbcu_stream_t stream);
int bbcu_fp32_BinaryToReal_Backward(const float *dev_dy_buf, float *dev_dx_buf, int node_mux_size, int frame_mux_size, int y_node_size,
                                    int x_frame_stride, int y_frame_size, int y_frame_stride, bbcu_stream_t stream);

/* ------------------------------------------------------------------ Convolution lowering (include/bbcu/bbcu.h:949-1186).
 * Lowering multiplies the frame axis by the output pixels: output frame = input frame * (output_h * output_w) + oy * output_w + ox.
 * border_mode: 0 constant (border_value; 0 for bit frames), 1 reflect, 2 reflect_101, 3 replicate, 4 wrap
 * (include/bb/ConvolutionIm2Col.h:253-288).  Results follow the reference's CPU branches; strides are in elements
 * (floats / 32-frame words). */
/* bbcu_fp32_Im2Col_Forward, bbcu.h:1076-1097: y[(c*fh + fy)*fw + fx][fo] = x[(c*ih + iy)*iw + ix][fi]. */
int bbcu_fp32_Im2Col_Forward(const float *dev_x_buf, float *dev_y_buf, int x_stride, int y_stride, int x_offset, int y_offset,
                             int input_frame_size, int input_frame_stride, int input_w_size, int input_h_size, int input_c_size,
                             int output_w_size, int output_h_size, int output_frame_stride, int filter_w_size, int filter_h_size,
                             int border_mode, float border_value, bbcu_stream_t stream);
/* bbcu_bit_Im2Col_Forward, bbcu.h:1099-1119.  Keeps a table of a few KiB per (geometry) in the stream's heap scratch: the first call
 * on a stream allocates (outside of stream capture); a heap that declines it is answered by slower kernels, not by an error. */
int bbcu_bit_Im2Col_Forward(const int *dev_x_buf, int *dev_y_buf, int x_stride, int y_stride, int x_offset, int y_offset,
                            int input_frame_size, int input_frame_stride, int input_w_size, int input_h_size, int input_c_size,
                            int output_w_size, int output_h_size, int output_frame_stride, int filter_w_size, int filter_h_size,
                            int border_mode, bbcu_stream_t stream);
/* bbcu_fp32_Im2Col_Backward, bbcu.h:1122-1141: dx overwritten; only in-image positions receive gradient
 * (include/bb/ConvolutionIm2Col.h:439-482). */
int bbcu_fp32_Im2Col_Backward(const float *dev_dy_buf, float *dev_dx_buf, int x_stride, int y_stride, int x_offset, int y_offset,
                              int input_frame_size, int input_frame_stride, int input_w_size, int input_h_size, int input_c_size,
                              int output_w_size, int output_h_size, int output_frame_stride, int filter_w_size, int filter_h_size,
                              bbcu_stream_t stream);
/* bbcu_fp32_Col2Im_Forward / bbcu_bit_Col2Im_Forward / bbcu_fp32_Col2Im_Backward, bbcu.h:1148-1186:
 * y[c*h*w + xy][fo] = x[c][fo*h*w + xy]; input_frame_stride belongs to the [c][...] side in all three. */
int bbcu_fp32_Col2Im_Forward(const float *dev_x_buf, float *dev_y_buf, int w_size, int h_size, int c_size, int input_frame_stride,
                             int output_frame_size, int output_frame_stride, bbcu_stream_t stream);
int bbcu_bit_Col2Im_Forward(const int *dev_x_buf, int *dev_y_buf, int w_size, int h_size, int c_size, int input_frame_stride,
                            int output_frame_size, int output_frame_stride, bbcu_stream_t stream);
int bbcu_fp32_Col2Im_Backward(const float *dev_dy_buf, float *dev_dx_buf, int w_size, int h_size, int c_size, int input_frame_stride,
                              int output_frame_size, int output_frame_stride, bbcu_stream_t stream);
/* bbcu_fp32_MaxPooling_Forward, bbcu.h:949-964: windows of filter_h x filter_w with the same stride, output size rounded up;
 * the first maximum wins; dev_argmax_buf (may be NULL) receives the winner's ordinal among the window's in-image positions
 * (include/bb/MaxPooling.h:286-322). */
int bbcu_fp32_MaxPooling_Forward(const float *dev_x_buf, float *dev_y_buf, int *dev_argmax_buf, int filter_h_size, int filter_w_size,
                                 int input_w_size, int input_h_size, int output_w_size, int output_h_size, int c_size, int frame_size,
                                 int frame_stride, bbcu_stream_t stream);
/* bbcu_bit_MaxPooling_Forward, bbcu.h:966-980: OR of the window. */
int bbcu_bit_MaxPooling_Forward(const int *dev_x_buf, int *dev_y_buf, int filter_h_size, int filter_w_size, int input_w_size,
                                int input_h_size, int output_w_size, int output_h_size, int c_size, int frame_size, int frame_stride,
                                bbcu_stream_t stream);
/* bbcu_fp32_MaxPooling_Backward, bbcu.h:983-998: dx = dy at the argmax position, 0 elsewhere. */
int bbcu_fp32_MaxPooling_Backward(const int *dev_argmax_buf, const float *dev_dy_buf, float *dev_dx_buf, int filter_h_size, int filter_w_size,
                                  int input_w_size, int input_h_size, int output_w_size, int output_h_size, int c_size, int frame_size,
                                  int frame_stride, bbcu_stream_t stream);
/* bbcu_bit_fp32_MaxPooling_Backward, bbcu.h:1000-1016: dev_x_buf is the bit layer's forward INPUT; the first set bit of a window
 * takes the gradient (include/bb/MaxPooling.h:681-708). */
int bbcu_bit_fp32_MaxPooling_Backward(const int *dev_x_buf, const float *dev_dy_buf, float *dev_dx_buf, int filter_h_size, int filter_w_size,
                                      int input_w_size, int input_h_size, int output_w_size, int output_h_size, int c_size, int frame_size,
                                      int forward_frame_stride, int backward_frame_stride, bbcu_stream_t stream);

/* ------------------------------------------------------------------ Additive: frame-sharded (multi-GPU) building blocks.
 * No counterpart in the reference (it has no multi-device path, include/bb/Memory.h:215-216).  A rank holds a contiguous frame
 * shard; these split the batch-norm operators at the points where per-node sums over ALL frames are needed, so the caller can
 * all-reduce `dev_sums` ([node_size][2] fp64) between the two halves.  total_frame_size is the global frame count. */
int bbcu_fp32_DifferentiableLut6_ForwardStats(const float *dev_x_buf, float *dev_y_buf, const int *dev_input_index, const float *dev_W,
                                              double *dev_sums, float unbinarize_bias, int node_size, int frame_size, int frame_stride,
                                              int lut_binarize, int binary_mode, bbcu_stream_t stream);
int bbcu_fp32_DifferentiableLut6_ForwardNormalize(float *dev_y_buf, const double *dev_sums, float *dev_mean_buf, float *dev_rstd_buf,
                                                  float *dev_running_mean_buf, float *dev_running_var_buf,
                                                  float gamma, float beta, float momentum, int node_size, int frame_size, int frame_stride,
                                                  long long total_frame_size, int binary_mode, bbcu_stream_t stream);
int bbcu_fp32_DifferentiableLut6_BackwardStats(const float *dev_x_buf, const float *dev_dy_buf, const int *dev_input_index, const float *dev_W,
                                               const float *dev_mean_buf, const float *dev_rstd_buf, double *dev_sums,
                                               float gamma, float beta, float unbinarize_bias, int node_size, int frame_size, int frame_stride,
                                               int lut_binarize, int binary_mode, bbcu_stream_t stream);
/* Same sums as ..._BackwardStats, taken from the layer's own training OUTPUT y instead of re-evaluating the LUT (non-binary mode
 * only; binary_mode != 0 is rejected): where 0 < y < 1 the pre-activation value is (y - beta) / gamma, elsewhere the gradient is
 * masked.  A stream over y and dy (8 bytes per node-frame). */
int bbcu_fp32_DifferentiableLut6_BackwardStatsFromOutput(const float *dev_y_buf, const float *dev_dy_buf, const float *dev_rstd_buf,
                                                         double *dev_sums, float gamma, float beta, int node_size, int frame_size,
                                                         int frame_stride, int binary_mode, bbcu_stream_t stream);
int bbcu_fp32_DifferentiableLut6_BackwardApply(const float *dev_x_buf, const float *dev_dy_buf, float *dev_dx_buf,
                                               const int *dev_input_index, const float *dev_W, float *dev_dW,
                                               const float *dev_mean_buf, const float *dev_rstd_buf, const double *dev_sums,
                                               float *dev_dmean_tmp, float *dev_dvar_tmp,
                                               float gamma, float beta, float unbinarize_bias, int input_node_size, int output_node_size,
                                               int frame_size, int frame_stride, long long total_frame_size,
                                               int lut_binarize, int binary_mode, bbcu_stream_t stream);

/* ------------------------------------------------------------------ Additive: a training forward that allocates nothing.
 * No counterpart in the reference.  Same arguments and results as bbcu_fp32_DifferentiableLut6_ForwardTraining, for callers that
 * cannot tolerate a cudaMalloc inside the call (a pre-planned device-memory budget, or a latency path that must not take
 * cudaMalloc's implicit device synchronisation): the per-node fp64 sums live in a fixed 1 MiB array inside the library's device
 * image instead of heap scratch.  node_size above ..._MaxNodes() (65536) returns BBCU_ERR_TOO_LARGE.  All calls on a device share
 * that array: calls whose GPU work may overlap race, so keep them on one stream.  The first call on each device resolves the
 * array's address and should be made outside of stream capture. */
int bbcu_fp32_DifferentiableLut6_ForwardTraining_NoAlloc(const float *dev_x_buf, float *dev_y_buf, const int *dev_input_index, const float *dev_W,
                                                         float *dev_mean_buf, float *dev_rstd_buf, float *dev_running_mean_buf,
                                                         float *dev_running_var_buf, float gamma, float beta, float momentum,
                                                         float unbinarize_bias, int node_size, int frame_size, int frame_stride,
                                                         int lut_binarize, int binary_mode, bbcu_stream_t stream);
int bbcu_fp32_DifferentiableLut6_ForwardTraining_NoAlloc_MaxNodes(void);

#ifdef __cplusplus
}
#endif
#endif /* BBCU_B200_H */
