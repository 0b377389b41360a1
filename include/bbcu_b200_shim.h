/* bbcu_b200_shim.h -- the reference-side binding: BinaryBrain's own operator names, forwarded to libbbcu_b200.so.
 *
 * For a BinaryBrain (ryuz/BinaryBrain v4.3.2) maintainer.  Include this header at the END of include/bbcu/bbcu.h and link
 * libbbcu_b200.so in place of cuda/StochasticLut.cu, DifferentiableLut.cu, BinaryLut6.cu, StochasticBatchNormalization.cu,
 * LocalHeap.cu, Manager.cu, OptimizerAdam.cu, Im2Col.cu, Col2Im.cu, MaxPooling.cu, BinaryToReal.cu, LossMeanSquaredError.cu and the
 * Vector clamp / set kernels.  bbcu.h keeps its declarations; the inline functions below are their definitions, so the call sites
 * in include/bb/DifferentiableLutN.h:633,662,697,725,919,943,1075,1126, StochasticLutN.h:463,487,599,643, BinaryLutN.h:307,
 * StochasticBatchNormalization.h:378-412,639,710, Memory.h, OptimizerAdam.h, ConvolutionIm2Col.h, ConvolutionCol2Im.h and
 * MaxPooling.h compile unchanged.  The LUT operators are templates on the LUT width N there; N == 6 forwards to the C symbol
 * and any other N fails to compile with a message.
 *
 * The C ABI is pulled into namespace bbcu_b200 because several of its symbols carry the same names as BinaryBrain's C++
 * declarations (a C-linkage function inside a namespace is still the plain C symbol for the linker).
 *
 * Error policy: BinaryBrain's operators always return 0 and exit(1) on a CUDA error (include/bbcu/bbcu_util.h:17-36).  Here a
 * non-zero status goes through BB_ASSERT, i.e. an assertion or, under BB_ASSERT_EXCEPTION, an exception.
 */
#ifndef BBCU_B200_SHIM_H
#define BBCU_B200_SHIM_H

#include <stddef.h>
#include <cuda_runtime.h>

namespace bbcu_b200 {
#include "bbcu_b200.h"
}
using bbcu_b200::bbcu_stream_t;

inline int bbcu_b200_shim_check(int status)
{
#ifdef BB_ASSERT
    BB_ASSERT(status == 0);
#endif
    return status;
}

/* bool in BinaryBrain (include/bbcu/bbcu.h:53-55), int in the C ABI */
inline void bbcu_SetHostOnly(bool hostOnly) { bbcu_b200::bbcu_SetHostOnly(hostOnly ? 1 : 0); }
inline bool bbcu_IsHostOnly(void) { return bbcu_b200::bbcu_IsHostOnly() != 0; }
inline bool bbcu_IsDeviceAvailable(void) { return bbcu_b200::bbcu_IsDeviceAvailable() != 0; }

inline int bbcu_GetDeviceCount(void) { return bbcu_b200::bbcu_GetDeviceCount(); }

inline int bbcu_GetDevice(void) { return bbcu_b200::bbcu_GetDevice(); }

inline void bbcu_SetDevice(int device) { bbcu_b200::bbcu_SetDevice(device); }

inline void  * bbcu_LocalHeap_Malloc(size_t size) { return bbcu_b200::bbcu_LocalHeap_Malloc(size); }

inline void bbcu_LocalHeap_Free(void * ptr) { bbcu_b200::bbcu_LocalHeap_Free(ptr); }

inline size_t bbcu_LocalHeap_GetMaxAllocSize(void) { return bbcu_b200::bbcu_LocalHeap_GetMaxAllocSize(); }

inline size_t bbcu_LocalHeap_GetAllocatedSize(void) { return bbcu_b200::bbcu_LocalHeap_GetAllocatedSize(); }

inline void bbcu_LocalHeap_GarbageCollect(void) { bbcu_b200::bbcu_LocalHeap_GarbageCollect(); }

template <int N> inline int bbcu_fp32_StochasticLut_Forward(const float * dev_x_buf, float * dev_y_buf, const int * dev_input_index, const float *
        dev_W, int node_size, int frame_size, int frame_stride, int input_binary, int lut_binarize, float unbinarize_bias, cudaStream_t streamId)
{
    static_assert(N == 6, "libbbcu_b200 provides the 6-input LUT only");
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_StochasticLut6_Forward(dev_x_buf, dev_y_buf, dev_input_index, dev_W, node_size, frame_size,
        frame_stride, input_binary, lut_binarize, unbinarize_bias, (bbcu_stream_t)streamId));
}

template <int N> inline int bbcu_bit_fp32_StochasticLut_Forward(const int * dev_x_buf, float * dev_y_buf, const int * dev_input_index, const float *
        dev_W, int node_size, int frame_size, int frame_stride, int bin_frame_stride, int lut_binarize, float unbinarize_bias, cudaStream_t streamId)
{
    static_assert(N == 6, "libbbcu_b200 provides the 6-input LUT only");
    return bbcu_b200_shim_check(bbcu_b200::bbcu_bit_fp32_StochasticLut6_Forward(dev_x_buf, dev_y_buf, dev_input_index, dev_W, node_size, frame_size,
        frame_stride, bin_frame_stride, lut_binarize, unbinarize_bias, (bbcu_stream_t)streamId));
}

template <int N> inline int bbcu_bit_bit_fp32_StochasticLut_Forward(const int * dev_x_buf, int * dev_y_buf, const int * dev_input_index, const float *
        dev_W, int node_size, int frame_size, int frame_stride, int lut_binarize, float unbinarize_bias, cudaStream_t streamId)
{
    static_assert(N == 6, "libbbcu_b200 provides the 6-input LUT only");
    return bbcu_b200_shim_check(bbcu_b200::bbcu_bit_bit_fp32_StochasticLut6_Forward(dev_x_buf, dev_y_buf, dev_input_index, dev_W, node_size,
        frame_size, frame_stride, lut_binarize, unbinarize_bias, (bbcu_stream_t)streamId));
}

template <int N> inline int bbcu_fp32_StochasticLut_Backward(const float * dev_x_buf, const float * dev_dy_buf, float * dev_dx_buf, float *
        dev_dx_tmp, const int * dev_input_index, const int * dev_reverse_index, const float * dev_W, float * dev_dW, int reverse_index_stride, int
        input_node_size, int output_node_size, int frame_size, int frame_stride, int tmp_frame_size, int tmp_frame_stride, int input_binary, int
        lut_binarize, float unbinarize_bias, cudaStream_t streamId)
{
    static_assert(N == 6, "libbbcu_b200 provides the 6-input LUT only");
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_StochasticLut6_Backward(dev_x_buf, dev_dy_buf, dev_dx_buf, dev_dx_tmp, dev_input_index,
        dev_reverse_index, dev_W, dev_dW, reverse_index_stride, input_node_size, output_node_size, frame_size, frame_stride, tmp_frame_size,
        tmp_frame_stride, input_binary, lut_binarize, unbinarize_bias, (bbcu_stream_t)streamId));
}

template <int N> inline int bbcu_bit_fp32_StochasticLut_Backward(const int * dev_x_buf, const float * dev_dy_buf, float * dev_dx_buf, float *
        dev_dx_tmp, const int * dev_input_index, const int * dev_reverse_index, const float * dev_W, float * dev_dW, int reverse_index_stride, int
        input_node_size, int output_node_size, int frame_size, int frame_stride, int bin_frame_stride, int tmp_frame_size, int tmp_frame_stride, int
        lut_binarize, float unbinarize_bias, cudaStream_t streamId)
{
    static_assert(N == 6, "libbbcu_b200 provides the 6-input LUT only");
    return bbcu_b200_shim_check(bbcu_b200::bbcu_bit_fp32_StochasticLut6_Backward(dev_x_buf, dev_dy_buf, dev_dx_buf, dev_dx_tmp, dev_input_index,
        dev_reverse_index, dev_W, dev_dW, reverse_index_stride, input_node_size, output_node_size, frame_size, frame_stride, bin_frame_stride,
        tmp_frame_size, tmp_frame_stride, lut_binarize, unbinarize_bias, (bbcu_stream_t)streamId));
}

template <int N> inline int bbcu_fp32_DifferentiableLutN_ForwardTraining(const float * dev_x_buf, float * dev_y_buf, const int * dev_input_index,
        const float * dev_W, float * dev_mean_buf, float * dev_rstd_buf, float * dev_running_mean_buf, float * dev_running_var_buf, float gamma, float
        beta, float momentum, float unbinarize_bias, int node_size, int frame_size, int frame_stride, int lut_binarize, int binary_mode, cudaStream_t
        streamId)
{
    static_assert(N == 6, "libbbcu_b200 provides the 6-input LUT only");
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_DifferentiableLut6_ForwardTraining(dev_x_buf, dev_y_buf, dev_input_index, dev_W, dev_mean_buf,
        dev_rstd_buf, dev_running_mean_buf, dev_running_var_buf, gamma, beta, momentum, unbinarize_bias, node_size, frame_size, frame_stride,
        lut_binarize, binary_mode, (bbcu_stream_t)streamId));
}

template <int N> inline int bbcu_bit_fp32_DifferentiableLutN_ForwardTraining(const int * dev_x_buf, int * dev_y_buf, const int * dev_input_index,
        const float * dev_W, float * dev_mean_buf, float * dev_rstd_buf, float * dev_running_mean_buf, float * dev_running_var_buf, float gamma, float
        beta, float momentum, float unbinarize_bias, int node_size, int frame_size, int frame_stride, int lut_binarize, cudaStream_t streamId)
{
    static_assert(N == 6, "libbbcu_b200 provides the 6-input LUT only");
    return bbcu_b200_shim_check(bbcu_b200::bbcu_bit_fp32_DifferentiableLut6_ForwardTraining(dev_x_buf, dev_y_buf, dev_input_index, dev_W,
        dev_mean_buf, dev_rstd_buf, dev_running_mean_buf, dev_running_var_buf, gamma, beta, momentum, unbinarize_bias, node_size, frame_size,
        frame_stride, lut_binarize, (bbcu_stream_t)streamId));
}

template <int N> inline int bbcu_fp32_DifferentiableLutN_ForwardInference(const float * dev_x_buf, float * dev_y_buf, const int * dev_input_index,
        const float * dev_W, const float * dev_running_mean_buf, const float * dev_running_var_buf, float gamma, float beta, float unbinarize_bias,
        int node_size, int frame_size, int frame_stride, int lut_binarize, int binary_mode, cudaStream_t streamId)
{
    static_assert(N == 6, "libbbcu_b200 provides the 6-input LUT only");
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_DifferentiableLut6_ForwardInference(dev_x_buf, dev_y_buf, dev_input_index, dev_W,
        dev_running_mean_buf, dev_running_var_buf, gamma, beta, unbinarize_bias, node_size, frame_size, frame_stride, lut_binarize, binary_mode,
        (bbcu_stream_t)streamId));
}

template <int N> inline int bbcu_bit_fp32_DifferentiableLutN_ForwardInference(const int * dev_x_buf, int * dev_y_buf, const int * dev_input_index,
        const float * dev_W, const float * dev_running_mean_buf, const float * dev_running_var_buf, float gamma, float beta, float unbinarize_bias,
        int node_size, int frame_size, int frame_stride, int lut_binarize, cudaStream_t streamId)
{
    static_assert(N == 6, "libbbcu_b200 provides the 6-input LUT only");
    return bbcu_b200_shim_check(bbcu_b200::bbcu_bit_fp32_DifferentiableLut6_ForwardInference(dev_x_buf, dev_y_buf, dev_input_index, dev_W,
        dev_running_mean_buf, dev_running_var_buf, gamma, beta, unbinarize_bias, node_size, frame_size, frame_stride, lut_binarize,
        (bbcu_stream_t)streamId));
}

template <int N> inline int bbcu_fp32_DifferentiableLutN_Backward(const float * dev_x_buf, const float * dev_dy_buf, float * dev_dx_buf, float *
        dev_dx_tmp, const int * dev_input_index, const int * dev_reverse_index, const float * dev_W, float * dev_dW, const float * dev_mean_buf, const
        float * dev_rstd_buf, float * dev_dmean_tmp, float * dev_dvar_tmp, float gamma, float beta, float unbinarize_bias, int reverse_index_stride,
        int input_node_size, int output_node_size, int frame_size, int frame_stride, int tmp_frame_size, int tmp_frame_stride, int lut_binarize, int
        binary_mode, cudaStream_t streamId)
{
    static_assert(N == 6, "libbbcu_b200 provides the 6-input LUT only");
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_DifferentiableLut6_Backward(dev_x_buf, dev_dy_buf, dev_dx_buf, dev_dx_tmp, dev_input_index,
        dev_reverse_index, dev_W, dev_dW, dev_mean_buf, dev_rstd_buf, dev_dmean_tmp, dev_dvar_tmp, gamma, beta, unbinarize_bias, reverse_index_stride,
        input_node_size, output_node_size, frame_size, frame_stride, tmp_frame_size, tmp_frame_stride, lut_binarize, binary_mode,
        (bbcu_stream_t)streamId));
}

template <int N> inline int bbcu_bit_fp32_DifferentiableLutN_Backward(const int * dev_x_buf, const float * dev_dy_buf, float * dev_dx_buf, float *
        dev_dx_tmp, const int * dev_input_index, const int * dev_reverse_index, const float * dev_W, float * dev_dW, const float * dev_mean_buf, const
        float * dev_rstd_buf, float * dev_dmean_tmp, float * dev_dvar_tmp, float gamma, float beta, float unbinarize_bias, int reverse_index_stride,
        int input_node_size, int output_node_size, int frame_size, int frame_stride, int x_frame_stride, int tmp_frame_size, int tmp_frame_stride, int
        lut_binarize, cudaStream_t streamId)
{
    static_assert(N == 6, "libbbcu_b200 provides the 6-input LUT only");
    return bbcu_b200_shim_check(bbcu_b200::bbcu_bit_fp32_DifferentiableLut6_Backward(dev_x_buf, dev_dy_buf, dev_dx_buf, dev_dx_tmp, dev_input_index,
        dev_reverse_index, dev_W, dev_dW, dev_mean_buf, dev_rstd_buf, dev_dmean_tmp, dev_dvar_tmp, gamma, beta, unbinarize_bias, reverse_index_stride,
        input_node_size, output_node_size, frame_size, frame_stride, x_frame_stride, tmp_frame_size, tmp_frame_stride, lut_binarize,
        (bbcu_stream_t)streamId));
}

inline int bbcu_fp32_StochasticBatchNormalization_ForwardTraining(const float * dev_x_buf, float * dev_y_buf, float * dev_mean_buf, float *
        dev_rstd_buf, float * dev_running_mean_buf, float * dev_running_var_buf, float gamma, float beta, float momentum, int node_size, int
        frame_size, int frame_stride, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_StochasticBatchNormalization_ForwardTraining(dev_x_buf, dev_y_buf, dev_mean_buf, dev_rstd_buf,
        dev_running_mean_buf, dev_running_var_buf, gamma, beta, momentum, node_size, frame_size, frame_stride, (bbcu_stream_t)streamId));
}

inline int bbcu_fp32_StochasticBatchNormalization_ReForward(const float * dev_x_buf, float * dev_y_buf, const float * dev_mean_buf, const float *
        dev_rstd_buf, float gamma, float beta, int node_size, int frame_size, int frame_stride, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_StochasticBatchNormalization_ReForward(dev_x_buf, dev_y_buf, dev_mean_buf, dev_rstd_buf, gamma,
        beta, node_size, frame_size, frame_stride, (bbcu_stream_t)streamId));
}

inline int bbcu_fp32_StochasticBatchNormalization_ForwardInference(const float * dev_x_buf, float * dev_y_buf, const float * dev_running_mean_buf,
        const float * dev_running_var_buf, float gamma, float beta, int node_size, int frame_size, int frame_stride, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_StochasticBatchNormalization_ForwardInference(dev_x_buf, dev_y_buf, dev_running_mean_buf,
        dev_running_var_buf, gamma, beta, node_size, frame_size, frame_stride, (bbcu_stream_t)streamId));
}

inline int bbcu_fp32_StochasticBatchNormalization_Backward(const float * dev_x_buf, const float * dev_dy_buf, float * dev_dx_buf, const float *
        dev_mean_buf, const float * dev_rstd_buf, float gamma, float reciprocal_frame_size, int node_size, int frame_size, int frame_stride, int
        x_frame_stride, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_StochasticBatchNormalization_Backward(dev_x_buf, dev_dy_buf, dev_dx_buf, dev_mean_buf,
        dev_rstd_buf, gamma, reciprocal_frame_size, node_size, frame_size, frame_stride, x_frame_stride, (bbcu_stream_t)streamId));
}

inline int bbcu_bit_BinatyLut6_Forward(const int * dev_x_buf, int * dev_y_buf, const int * dev_input_index, const int * dev_table, int node_size, int
        frame_size, int frame_stride, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_bit_BinatyLut6_Forward(dev_x_buf, dev_y_buf, dev_input_index, dev_table, node_size, frame_size,
        frame_stride, (bbcu_stream_t)streamId));
}

inline int bbcu_int32_FrameBufferCopy(int * dev_dst_buf, const int * dev_src_buf, int node_size, int dst_node_offset, int src_node_offset,
        int frame_size, int dst_frame_offset, int src_frame_offset, int dst_frame_stride, int src_frame_stride, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_int32_FrameBufferCopy(dev_dst_buf, dev_src_buf, node_size, dst_node_offset, src_node_offset,
            frame_size, dst_frame_offset, src_frame_offset, dst_frame_stride, src_frame_stride, (bbcu_stream_t)streamId));
}

/* a template on the value type in BinaryBrain (include/bbcu/bbcu.h:247-258); float is the one instance its headers use */
template <typename T> inline int bbcu_ConvBitToReal(const int * dev_x_buf, T * dev_y_buf, T value0, T value1, int node_size, int frame_size,
        int x_frame_stride, int y_frame_stride, cudaStream_t streamId)
{
    static_assert(sizeof(T) == sizeof(float) && T(0.5) > T(0), "libbbcu_b200 provides the float conversion only");
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_ConvBitToReal(dev_x_buf, (float *)dev_y_buf, (float)value0, (float)value1, node_size,
            frame_size, x_frame_stride, y_frame_stride, (bbcu_stream_t)streamId));
}

/* Leave these two out (define BBCU_B200_SHIM_NO_VECTOR) when cuda/Vector.cu stays in the build for the tensor arithmetic. */
#ifndef BBCU_B200_SHIM_NO_VECTOR
inline int bbcu_fp32_Vector_clamp(float * dev_dst, const float * dev_src, float lo, float hi, int size, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_Vector_clamp(dev_dst, dev_src, lo, hi, size, (bbcu_stream_t)streamId));
}

inline int bbcu_fp32_Vector_set(float * dev_dst, float a, int size, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_Vector_set(dev_dst, a, size, (bbcu_stream_t)streamId));
}
#endif

inline int bbcu_fp32_OptimizerAdam(int size, const int * dev_size_table, float *const * dev_params_buf_table, float *const * dev_grads_buf_table,
        float *const * dev_m_buf_table, float *const * dev_v_buf_table, float lr_t, float beta1, float beta2, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_OptimizerAdam(size, dev_size_table, dev_params_buf_table, dev_grads_buf_table, dev_m_buf_table,
        dev_v_buf_table, lr_t, beta1, beta2, (bbcu_stream_t)streamId));
}

inline int bbcu_fp32_LossMeanSquaredError(const float * dev_y_buf, const float * dev_t_buf, float * dev_dy_buf, double * dev_loss_buf, int
        loss_buf_size, int node_size, int frame_size, int frame_stride, float grad_reduction, double loss_reduction, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_LossMeanSquaredError(dev_y_buf, dev_t_buf, dev_dy_buf, dev_loss_buf, loss_buf_size, node_size,
        frame_size, frame_stride, grad_reduction, loss_reduction, (bbcu_stream_t)streamId));
}

inline int bbcu_bit_fp32_BinaryToReal_Forward(const int * dev_x_buf, float * dev_y_buf, int node_mux_size, int frame_mux_size, int y_node_size, int
        x_frame_stride, int y_frame_size, int y_frame_stride, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_bit_fp32_BinaryToReal_Forward(dev_x_buf, dev_y_buf, node_mux_size, frame_mux_size, y_node_size,
        x_frame_stride, y_frame_size, y_frame_stride, (bbcu_stream_t)streamId));
}

inline int bbcu_fp32_BinaryToReal_Forward(const float * dev_x_buf, float * dev_y_buf, int node_mux_size, int frame_mux_size, int y_node_size, int
        x_frame_stride, int y_frame_size, int y_frame_stride, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_BinaryToReal_Forward(dev_x_buf, dev_y_buf, node_mux_size, frame_mux_size, y_node_size,
        x_frame_stride, y_frame_size, y_frame_stride, (bbcu_stream_t)streamId));
}

inline int bbcu_fp32_BinaryToReal_Backward(const float * dev_dy_buf, float * dev_dx_buf, int node_mux_size, int frame_mux_size, int y_node_size, int
        x_frame_stride, int y_frame_size, int y_frame_stride, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_BinaryToReal_Backward(dev_dy_buf, dev_dx_buf, node_mux_size, frame_mux_size, y_node_size,
        x_frame_stride, y_frame_size, y_frame_stride, (bbcu_stream_t)streamId));
}

inline int bbcu_fp32_Im2Col_Forward(const float * dev_x_buf, float * dev_y_buf, int x_stride, int y_stride, int x_offset, int y_offset, int
        input_frame_size, int input_frame_stride, int input_w_size, int input_h_size, int input_c_size, int output_w_size, int output_h_size, int
        output_frame_stride, int filter_w_size, int filter_h_size, int border_mode, float border_value, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_Im2Col_Forward(dev_x_buf, dev_y_buf, x_stride, y_stride, x_offset, y_offset, input_frame_size,
        input_frame_stride, input_w_size, input_h_size, input_c_size, output_w_size, output_h_size, output_frame_stride, filter_w_size, filter_h_size,
        border_mode, border_value, (bbcu_stream_t)streamId));
}

inline int bbcu_bit_Im2Col_Forward(const int * dev_x_buf, int * dev_y_buf, int x_stride, int y_stride, int x_offset, int y_offset, int
        input_frame_size, int input_frame_stride, int input_w_size, int input_h_size, int input_c_size, int output_w_size, int output_h_size, int
        output_frame_stride, int filter_w_size, int filter_h_size, int border_mode, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_bit_Im2Col_Forward(dev_x_buf, dev_y_buf, x_stride, y_stride, x_offset, y_offset, input_frame_size,
        input_frame_stride, input_w_size, input_h_size, input_c_size, output_w_size, output_h_size, output_frame_stride, filter_w_size, filter_h_size,
        border_mode, (bbcu_stream_t)streamId));
}

inline int bbcu_fp32_Im2Col_Backward(const float * dev_dy_buf, float * dev_dx_buf, int x_stride, int y_stride, int x_offset, int y_offset, int
        input_frame_size, int input_frame_stride, int input_w_size, int input_h_size, int input_c_size, int output_w_size, int output_h_size, int
        output_frame_stride, int filter_w_size, int filter_h_size, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_Im2Col_Backward(dev_dy_buf, dev_dx_buf, x_stride, y_stride, x_offset, y_offset, input_frame_size,
        input_frame_stride, input_w_size, input_h_size, input_c_size, output_w_size, output_h_size, output_frame_stride, filter_w_size, filter_h_size,
        (bbcu_stream_t)streamId));
}

inline int bbcu_fp32_Col2Im_Forward(const float * dev_x_buf, float * dev_y_buf, int w_size, int h_size, int c_size, int input_frame_stride, int
        output_frame_size, int output_frame_stride, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_Col2Im_Forward(dev_x_buf, dev_y_buf, w_size, h_size, c_size, input_frame_stride,
        output_frame_size, output_frame_stride, (bbcu_stream_t)streamId));
}

inline int bbcu_bit_Col2Im_Forward(const int * dev_x_buf, int * dev_y_buf, int w_size, int h_size, int c_size, int input_frame_stride, int
        output_frame_size, int output_frame_stride, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_bit_Col2Im_Forward(dev_x_buf, dev_y_buf, w_size, h_size, c_size, input_frame_stride,
        output_frame_size, output_frame_stride, (bbcu_stream_t)streamId));
}

inline int bbcu_fp32_Col2Im_Backward(const float * dev_dy_buf, float * dev_dx_buf, int w_size, int h_size, int c_size, int input_frame_stride, int
        output_frame_size, int output_frame_stride, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_Col2Im_Backward(dev_dy_buf, dev_dx_buf, w_size, h_size, c_size, input_frame_stride,
        output_frame_size, output_frame_stride, (bbcu_stream_t)streamId));
}

inline int bbcu_fp32_MaxPooling_Forward(const float * dev_x_buf, float * dev_y_buf, int * dev_argmax_buf, int filter_h_size, int filter_w_size, int
        input_w_size, int input_h_size, int output_w_size, int output_h_size, int c_size, int frame_size, int frame_stride, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_MaxPooling_Forward(dev_x_buf, dev_y_buf, dev_argmax_buf, filter_h_size, filter_w_size,
        input_w_size, input_h_size, output_w_size, output_h_size, c_size, frame_size, frame_stride, (bbcu_stream_t)streamId));
}

inline int bbcu_bit_MaxPooling_Forward(const int * dev_x_buf, int * dev_y_buf, int filter_h_size, int filter_w_size, int input_w_size, int
        input_h_size, int output_w_size, int output_h_size, int c_size, int frame_size, int frame_stride, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_bit_MaxPooling_Forward(dev_x_buf, dev_y_buf, filter_h_size, filter_w_size, input_w_size, input_h_size,
        output_w_size, output_h_size, c_size, frame_size, frame_stride, (bbcu_stream_t)streamId));
}

inline int bbcu_fp32_MaxPooling_Backward(const int * dev_argmax_buf, const float * dev_dy_buf, float * dev_dx_buf, int filter_h_size, int
        filter_w_size, int input_w_size, int input_h_size, int output_w_size, int output_h_size, int c_size, int frame_size, int frame_stride,
        cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_fp32_MaxPooling_Backward(dev_argmax_buf, dev_dy_buf, dev_dx_buf, filter_h_size, filter_w_size,
        input_w_size, input_h_size, output_w_size, output_h_size, c_size, frame_size, frame_stride, (bbcu_stream_t)streamId));
}

inline int bbcu_bit_fp32_MaxPooling_Backward(const int * dev_x_buf, const float * dev_dy_buf, float * dev_dx_buf, int filter_h_size, int
        filter_w_size, int input_w_size, int input_h_size, int output_w_size, int output_h_size, int c_size, int frame_size, int forward_frame_stride,
        int backward_frame_stride, cudaStream_t streamId)
{
    return bbcu_b200_shim_check(bbcu_b200::bbcu_bit_fp32_MaxPooling_Backward(dev_x_buf, dev_dy_buf, dev_dx_buf, filter_h_size, filter_w_size,
        input_w_size, input_h_size, output_w_size, output_h_size, c_size, frame_size, forward_frame_stride, backward_frame_stride,
        (bbcu_stream_t)streamId));
}

#endif /* BBCU_B200_SHIM_H */
