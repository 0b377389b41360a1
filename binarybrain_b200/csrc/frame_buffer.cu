// FrameBuffer helpers on the device: the sub-block copy behind FrameBuffer::CopyTo (BinaryBrain include/bb/FrameBuffer.h:481-535,
// operator include/bbcu/bbcu.h:265-278, cuda/FrameBufferCopy.cu) and the bit -> fp32 conversion behind FrameBuffer::ConvertTo
// (include/bb/FrameBuffer.h:843-866, operator include/bbcu/bbcu.h:247-258, cuda/ConvBitToReal.cu).
//
// Both are pure HBM streams.  One CTA handles one row segment of 4096 words; a warp access is a whole 128-byte line (one word
// per lane), or 512 bytes with 128-bit accesses when both sides are 16-byte aligned.
#include "common.cuh"

namespace bb200 {

constexpr int kFbChunk = 4096;        // words per CTA

__global__ void __launch_bounds__(256)
k_frame_buffer_copy(int *__restrict__ dst, const int *__restrict__ src, int frame_words, long long dst_stride, long long src_stride, int chunks, int vec)
{
    const int node = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    int *d = dst + (size_t)node * dst_stride;
    const int *s = src + (size_t)node * src_stride;
    const int w0 = chunk * kFbChunk, w1 = min(frame_words, w0 + kFbChunk);
    if (vec) {
        // four 128-bit loads of a thread are in flight before its first store
        int4 v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int w = w0 + 4 * threadIdx.x + 1024 * k;
            if (w + 3 < w1) v[k] = __ldg(reinterpret_cast<const int4 *>(s + w));
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int w = w0 + 4 * threadIdx.x + 1024 * k;
            if (w + 3 < w1) *reinterpret_cast<int4 *>(d + w) = v[k];
            else for (int i = w; i < w1; ++i) d[i] = s[i];            // ragged end of the row segment (at most three words)
        }
    } else {
        for (int w = w0 + threadIdx.x; w < w1; w += 256) d[w] = __ldg(s + w);
    }
}

__global__ void __launch_bounds__(256)
k_conv_bit_to_real(const uint32_t *__restrict__ x, float *__restrict__ y, float value0, float value1, int frame_size, long long x_stride,
                   long long y_stride, int chunks, int vec)
{
    const int node = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    const uint32_t *xr = x + (size_t)node * x_stride;
    float *yr = y + (size_t)node * y_stride;
    const int f0 = chunk * kFbChunk, f1 = min(frame_size, f0 + kFbChunk);
    if (vec) {
        for (int f = f0 + 4 * threadIdx.x; f < f1; f += 1024) {
            const uint32_t w = __ldg(xr + (f >> 5)) >> (f & 31);          // f is a multiple of 4: the four bits sit in one word
            if (f + 3 < f1) {
                *reinterpret_cast<float4 *>(yr + f) = make_float4((w & 1u) ? value1 : value0, (w & 2u) ? value1 : value0, (w & 4u) ? value1 : value0,
                                                                  (w & 8u) ? value1 : value0);
            } else {
                for (int i = 0; f + i < f1; ++i) yr[f + i] = ((w >> i) & 1u) ? value1 : value0;
            }
        }
    } else {
        for (int f = f0 + threadIdx.x; f < f1; f += 256) yr[f] = ((__ldg(xr + (f >> 5)) >> (f & 31)) & 1u) ? value1 : value0;
    }
}

}   // namespace bb200

using namespace bb200;

extern "C" int bbcu_int32_FrameBufferCopy(int *dev_dst_buf, const int *dev_src_buf, int node_size, int dst_node_offset, int src_node_offset,
                                          int frame_size, int dst_frame_offset, int src_frame_offset, int dst_frame_stride, int src_frame_stride,
                                          bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(dev_dst_buf); BB200_REQUIRE_PTR(dev_src_buf);
    BB200_REQUIRE(node_size >= 0 && frame_size >= 0 && dst_node_offset >= 0 && src_node_offset >= 0 && dst_frame_offset >= 0 && src_frame_offset >= 0,
                  BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE((long long)dst_frame_offset + frame_size <= dst_frame_stride && (long long)src_frame_offset + frame_size <= src_frame_stride,
                  BBCU_ERR_BAD_STRIDE);
    if (node_size == 0 || frame_size == 0) return BBCU_OK;
    int *dst = dev_dst_buf + (size_t)dst_node_offset * dst_frame_stride + dst_frame_offset;
    const int *src = dev_src_buf + (size_t)src_node_offset * src_frame_stride + src_frame_offset;
    const int vec = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0 && dst_frame_stride % 4 == 0 && src_frame_stride % 4 == 0;
    const int chunks = (frame_size + kFbChunk - 1) / kFbChunk;
    BB200_REQUIRE((long long)node_size * chunks < (1LL << 31), BBCU_ERR_TOO_LARGE);
    k_frame_buffer_copy<<<node_size * chunks, 256, 0, as_stream(stream)>>>(dst, src, frame_size, dst_frame_stride, src_frame_stride, chunks, vec);
    return launch_status();
}

extern "C" int bbcu_fp32_ConvBitToReal(const int *dev_x_buf, float *dev_y_buf, float value0, float value1, int node_size, int frame_size,
                                       int x_frame_stride, int y_frame_stride, bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(dev_x_buf); BB200_REQUIRE_PTR(dev_y_buf);
    BB200_REQUIRE(node_size >= 0 && frame_size >= 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE((long long)x_frame_stride * 32 >= frame_size && y_frame_stride >= frame_size, BBCU_ERR_BAD_STRIDE);
    if (node_size == 0 || frame_size == 0) return BBCU_OK;
    const int vec = (reinterpret_cast<uintptr_t>(dev_y_buf) & 15) == 0 && y_frame_stride % 4 == 0;
    const int chunks = (frame_size + kFbChunk - 1) / kFbChunk;
    BB200_REQUIRE((long long)node_size * chunks < (1LL << 31), BBCU_ERR_TOO_LARGE);
    k_conv_bit_to_real<<<node_size * chunks, 256, 0, as_stream(stream)>>>(reinterpret_cast<const uint32_t *>(dev_x_buf), dev_y_buf, value0, value1,
                                                                           frame_size, x_frame_stride, y_frame_stride, chunks, vec);
    return launch_status();
}
