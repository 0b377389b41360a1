// bb::Memory / bb::Tensor_ / bb::FrameBuffer -- host-side containers in BinaryBrain's style over the
// bbcu_* C ABI.
//
// Same roles and layout as the reference's include/bb/Memory.h:45-823, Tensor.h and FrameBuffer.h:269-1720:
// a lazily mirrored host/device pair with dirty flags, fp32 / bit frame buffers that are node-major and
// frame-contiguous with rows padded to 256 bits (FrameBuffer.h:28-46,414-417).  Differences by design:
// device memory comes from the per-device caching heap of libbbcu_b200 (bbcu_LocalHeap_*), copies are
// cudaMemcpyAsync on the layer stream followed by one stream sync when the HOST side needs the data, and
// there are no ref-counted lock objects: Host()/Dev() return the pointer after making that side current.
#pragma once

#include <cuda_runtime_api.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <new>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "bbcu_b200.h"

#define BB_TYPE_BIT   (0x0000 + 1)
#define BB_TYPE_FP32  (0x0100 + 32)
#define BB_TYPE_INT32 (0x0200 + 32)

namespace bb {

using index_t   = std::int64_t;
using indices_t = std::vector<index_t>;

struct Bit {};   // tag type: one bit per frame, 32 frames per 32-bit word, LSB first

template <typename T> struct DataType;
template <> struct DataType<float>        { static constexpr int type = BB_TYPE_FP32;  static const char *Name() { return "fp32"; } };
template <> struct DataType<Bit>          { static constexpr int type = BB_TYPE_BIT;   static const char *Name() { return "bit"; } };
template <> struct DataType<std::int32_t> { static constexpr int type = BB_TYPE_INT32; static const char *Name() { return "int32"; } };

inline int DataType_GetBitSize(int type) { return type == BB_TYPE_BIT ? 1 : 32; }

inline index_t CalcShapeSize(indices_t const &shape)
{
    index_t n = 1;
    for (auto s : shape) n *= s;
    return n;
}

// BinaryBrain's BB_ASSERT under BB_ASSERT_EXCEPTION (include/bb/Assert.h:24-42): a C++ exception, never exit().
#define BB_ASSERT(cond) \
    do { if (!(cond)) { std::ostringstream os_; os_ << "BB_ASSERT(" #cond ") failed at " << __FILE__ << ":" << __LINE__; \
                        throw std::runtime_error(os_.str()); } } while (0)

inline void bbcu_check(int status, char const *what)
{
    if (status != 0) {
        throw std::runtime_error(std::string(what) + ": " + bbcu_b200_error_string(status));
    }
}
#define BBCU_CHECK(call) ::bb::bbcu_check((call), #call)

inline void cuda_check(cudaError_t e, char const *what)
{
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
#define BB_CUDA_CHECK(call) ::bb::cuda_check((call), #call)


class Manager
{
public:
    static bool IsDeviceAvailable() { return bbcu_IsDeviceAvailable() != 0; }
    static void SetHostOnly(bool h) { bbcu_SetHostOnly(h ? 1 : 0); }
    static int  GetDeviceCount()    { return bbcu_GetDeviceCount(); }
    static void SetDevice(int d)    { bbcu_SetDevice(d); }
    // The stream every layer enqueues on (default stream unless a caller installs another one).
    static cudaStream_t &Stream() { static cudaStream_t s = nullptr; return s; }
};


// Host/device mirrored byte buffer.  The host mirror of a buffer of kPinnedFrom bytes or more is page-locked (cudaMallocHost, as the
// reference's include/bbcu/bbcu_util.h:121 does for every host buffer) so that its transfers run at full PCIe rate and
// asynchronously; small buffers and processes without a device use plain heap memory.  Either side is materialised on first use:
// a frame buffer that only ever lives on the device (every activation of a training step) never allocates or clears host memory.
// A buffer that nothing has written yet reads as zeros on whichever side is asked for first.
class Memory
{
    static constexpr std::size_t kPinnedFrom = 64 * 1024;

    std::size_t     m_size = 0;
    std::uint8_t   *m_host = nullptr;
    bool            m_pinned = false;
    void           *m_dev = nullptr;
    bool            m_host_valid = false;   // host copy holds the current contents
    bool            m_dev_valid  = false;   // device copy holds the current contents; neither: the contents are zeros

    void release_host()
    {
        if (m_host) { if (m_pinned) bbcu_b200_host_free(m_host); else std::free(m_host); }
        m_host = nullptr;
        m_pinned = false;
    }
    bool want_pinned() const { return m_size >= kPinnedFrom && Manager::IsDeviceAvailable(); }
    void ensure_host()
    {
        if (m_host) return;
        if (want_pinned()) {
            m_host = static_cast<std::uint8_t *>(bbcu_b200_host_alloc(m_size));
            m_pinned = m_host != nullptr;
        }
        if (!m_host) m_host = static_cast<std::uint8_t *>(std::malloc(m_size ? m_size : 1));
        if (!m_host) throw std::bad_alloc();
    }
    // bring the host copy up to date: from the device when that holds the contents, zeros when nothing does
    void refresh_host(bool new_buf)
    {
        ensure_host();
        if (m_host_valid || new_buf) return;
        if (m_dev && m_dev_valid) {
            BB_CUDA_CHECK(cudaMemcpyAsync(m_host, m_dev, m_size, cudaMemcpyDeviceToHost, Manager::Stream()));
            BB_CUDA_CHECK(cudaStreamSynchronize(Manager::Stream()));
        } else {
            std::memset(m_host, 0, m_size);
        }
    }

public:
    Memory() {}
    explicit Memory(std::size_t size) { Resize(size); }
    Memory(Memory const &) = delete;
    Memory &operator=(Memory const &) = delete;
    ~Memory() { if (m_dev) bbcu_LocalHeap_Free(m_dev); release_host(); }

    void Resize(std::size_t size)
    {
        if (m_dev) { bbcu_LocalHeap_Free(m_dev); m_dev = nullptr; }
        release_host();
        m_size = size;
        m_host_valid = false;
        m_dev_valid  = false;
    }
    std::size_t GetSize() const { return m_size; }
    bool IsHostPinned() const { return m_host ? m_pinned : want_pinned(); }      // what the mirror is, or will be once it exists
    bool IsDeviceCurrent() const { return m_dev_valid; }

    // new_buf: the caller overwrites everything, so nothing is copied (reference: Lock(true)).
    void *Host(bool new_buf = false)
    {
        refresh_host(new_buf);
        m_host_valid = true;
        m_dev_valid  = false;
        return m_host;
    }
    void const *HostConst()
    {
        refresh_host(false);
        m_host_valid = true;
        return m_host;
    }
    void *Dev(bool new_buf = false)
    {
        DevConst(new_buf);
        m_host_valid = false;
        return m_dev;
    }
    void const *DevConst(bool new_buf = false)
    {
        BB_ASSERT(Manager::IsDeviceAvailable());     // no CPU fallback behind the operators
        if (!m_dev) {
            m_dev = bbcu_LocalHeap_Malloc(m_size);
            if (!m_dev) throw std::runtime_error("bbcu_LocalHeap_Malloc: device memory exhausted");
            m_dev_valid = false;
        }
        if (!m_dev_valid && !new_buf && m_size) {
            if (m_host && m_host_valid) {
                BB_CUDA_CHECK(cudaMemcpyAsync(m_dev, m_host, m_size, cudaMemcpyHostToDevice, Manager::Stream()));
                // a page-locked source is read by the copy engine after this call returns: the host side may write it again only once
                // the copy is done (a pageable source has been staged by the runtime already)
                if (m_pinned) BB_CUDA_CHECK(cudaStreamSynchronize(Manager::Stream()));
            } else {
                BB_CUDA_CHECK(cudaMemsetAsync(m_dev, 0, m_size, Manager::Stream()));
            }
        }
        m_dev_valid = true;
        return m_dev;
    }
};


// Dense typed tensor (parameters, statistics, tables).
template <typename T>
class Tensor_
{
    indices_t               m_shape;
    std::shared_ptr<Memory> m_mem = std::make_shared<Memory>();

public:
    Tensor_() {}
    explicit Tensor_(indices_t shape) { Resize(shape); }
    void Resize(indices_t shape) { m_shape = shape; m_mem->Resize(sizeof(T) * (std::size_t)CalcShapeSize(shape)); }
    void Resize(index_t n) { Resize(indices_t{n}); }
    indices_t GetShape() const { return m_shape; }
    index_t   GetSize()  const { return CalcShapeSize(m_shape); }
    T       *Host(bool new_buf = false) { return static_cast<T *>(m_mem->Host(new_buf)); }
    T const *HostConst() const          { return static_cast<T const *>(m_mem->HostConst()); }
    T       *Dev(bool new_buf = false)  { return static_cast<T *>(m_mem->Dev(new_buf)); }
    T const *DevConst() const           { return static_cast<T const *>(m_mem->DevConst()); }
    void Fill(T v) { T *p = Host(true); for (index_t i = 0; i < GetSize(); ++i) p[i] = v; }
    void FillZero() { std::memset(m_mem->Host(true), 0, m_mem->GetSize()); }
    T  operator()(index_t i, index_t j) const { return HostConst()[i * m_shape.back() + j]; }
    std::vector<T> ToVector() const { T const *p = HostConst(); return std::vector<T>(p, p + GetSize()); }
    void FromVector(std::vector<T> const &v) { BB_ASSERT((index_t)v.size() == GetSize()); std::memcpy(Host(true), v.data(), sizeof(T) * v.size()); }
};

using Tensor = Tensor_<float>;


// [node][frame] buffer of fp32 or bit frames.
class FrameBuffer
{
    index_t                 m_frame_size = 0;
    index_t                 m_frame_stride = 0;     // BYTES per node row (reference: GetFrameStride())
    indices_t               m_shape;
    int                     m_type = 0;
    std::shared_ptr<Memory> m_mem;

public:
    FrameBuffer() {}
    FrameBuffer(index_t frame_size, indices_t shape, int data_type, bool /*host_only*/ = false) { Resize(frame_size, shape, data_type); }

    // rows are padded to 256 bits (include/bb/FrameBuffer.h:414-417)
    static index_t CalcFrameStride(int data_type, index_t frame_size)
    {
        return ((frame_size * DataType_GetBitSize(data_type) + 255) / 256) * (256 / 8);
    }

    void Resize(index_t frame_size, indices_t shape, int data_type)
    {
        BB_ASSERT(data_type == BB_TYPE_FP32 || data_type == BB_TYPE_BIT);
        m_frame_size   = frame_size;
        m_frame_stride = CalcFrameStride(data_type, frame_size);
        m_shape        = shape;
        m_type         = data_type;
        m_mem          = std::make_shared<Memory>((std::size_t)(m_frame_stride * CalcShapeSize(shape)));
    }

    bool      Empty()          const { return !m_mem; }
    int       GetType()        const { return m_type; }
    index_t   GetFrameSize()   const { return m_frame_size; }
    index_t   GetFrameStride() const { return m_frame_stride; }
    index_t   GetNodeSize()    const { return CalcShapeSize(m_shape); }
    indices_t GetShape()       const { return m_shape; }
    bool      IsDeviceAvailable() const { return Manager::IsDeviceAvailable(); }

    void       *LockDeviceMemory(bool new_buf = false) { return m_mem->Dev(new_buf); }
    void const *LockDeviceMemoryConst() const          { return m_mem->DevConst(); }
    void       *LockMemory(bool new_buf = false)       { return m_mem->Host(new_buf); }
    void const *LockMemoryConst() const                { return m_mem->HostConst(); }

    void FillZero() { std::memset(m_mem->Host(true), 0, m_mem->GetSize()); }
    bool IsHostPinned() const { return m_mem && m_mem->IsHostPinned(); }

    // ---- copies and views (include/bb/FrameBuffer.h:372-395, 465-560, 843-900, 1370-1460).  Where the data is current on the
    // device the work is done there (bbcu_int32_FrameBufferCopy, bbcu_fp32_ConvBitToReal); otherwise on the host mirror.
    FrameBuffer Clone() const
    {
        FrameBuffer dst(m_frame_size, m_shape, m_type);
        CopyTo(dst);
        return dst;
    }

    // Block copy of frame_size frames x node_size nodes (0 = as many as fit).  Bit buffers: frame offsets and sizes are multiples of 32
    // on the device path; other bit ranges go through the host mirror bit by bit.
    void CopyTo(FrameBuffer &dst, index_t frame_size = 0, index_t src_frame_offset = 0, index_t dst_frame_offset = 0, index_t node_size = 0,
                index_t src_node_offset = 0, index_t dst_node_offset = 0) const
    {
        BB_ASSERT(dst.GetType() == GetType());
        if (node_size <= 0)  node_size  = std::min(dst.GetNodeSize() - dst_node_offset, GetNodeSize() - src_node_offset);
        if (frame_size <= 0) frame_size = std::min(dst.GetFrameSize() - dst_frame_offset, GetFrameSize() - src_frame_offset);
        BB_ASSERT(frame_size + src_frame_offset <= GetFrameSize() && frame_size + dst_frame_offset <= dst.GetFrameSize());
        BB_ASSERT(node_size + src_node_offset <= GetNodeSize() && node_size + dst_node_offset <= dst.GetNodeSize());
        const bool bit = m_type == BB_TYPE_BIT;
        const bool word_aligned = !bit || (frame_size % 32 == 0 && src_frame_offset % 32 == 0 && dst_frame_offset % 32 == 0);
        if (m_mem->IsDeviceCurrent() && word_aligned && Manager::IsDeviceAvailable()) {
            const index_t per = bit ? 32 : 1;
            BBCU_CHECK(bbcu_int32_FrameBufferCopy(static_cast<int *>(dst.m_mem->Dev()), static_cast<int const *>(m_mem->DevConst()), (int)node_size,
                                                  (int)dst_node_offset, (int)src_node_offset, (int)(frame_size / per), (int)(dst_frame_offset / per),
                                                  (int)(src_frame_offset / per), (int)(dst.m_frame_stride / 4), (int)(m_frame_stride / 4),
                                                  Manager::Stream()));
            return;
        }
        auto sp = static_cast<std::uint8_t const *>(m_mem->HostConst());
        auto dp = static_cast<std::uint8_t *>(dst.m_mem->Host());
        for (index_t n = 0; n < node_size; ++n) {
            auto srow = sp + (n + src_node_offset) * m_frame_stride;
            auto drow = dp + (n + dst_node_offset) * dst.m_frame_stride;
            if (!bit) {
                std::memcpy(drow + 4 * dst_frame_offset, srow + 4 * src_frame_offset, 4 * (std::size_t)frame_size);
            } else {
                for (index_t f = 0; f < frame_size; ++f) {
                    const index_t sf = f + src_frame_offset, df = f + dst_frame_offset;
                    const std::uint32_t b = (reinterpret_cast<std::uint32_t const *>(srow)[sf >> 5] >> (sf & 31)) & 1u;
                    auto &w = reinterpret_cast<std::uint32_t *>(drow)[df >> 5];
                    w = (w & ~(1u << (df & 31))) | (b << (df & 31));
                }
            }
        }
    }

    // `size` frames from `offset` on, as a new buffer (FrameBuffer.h:1370-1405)
    FrameBuffer FrameRange(index_t size, index_t offset = 0) const
    {
        BB_ASSERT(offset >= 0 && offset < m_frame_size && size >= 0 && size <= m_frame_size - offset);
        FrameBuffer dst(size, m_shape, m_type);
        if (size > 0) CopyTo(dst, size, offset, 0);
        return dst;
    }

    // `size` nodes from `offset` on, as a new 1-D buffer (FrameBuffer.h:1408-1424)
    FrameBuffer Range(index_t size, index_t offset = 0) const
    {
        BB_ASSERT(offset >= 0 && offset < GetNodeSize() && size >= 0 && size <= GetNodeSize() - offset);
        FrameBuffer dst(m_frame_size, {size}, m_type);
        if (size > 0 && m_frame_size > 0) CopyTo(dst, m_frame_size, 0, 0, size, offset, 0);
        return dst;
    }

    // the nodes of `buf` appended to this buffer's (FrameBuffer.h:1427-1455)
    FrameBuffer Concatenate(FrameBuffer const &buf) const
    {
        BB_ASSERT(buf.GetType() == GetType() && buf.m_frame_size == m_frame_size);
        FrameBuffer dst(m_frame_size, {GetNodeSize() + buf.GetNodeSize()}, m_type);
        if (m_frame_size > 0) {
            CopyTo(dst, m_frame_size, 0, 0, GetNodeSize(), 0, 0);
            buf.CopyTo(dst, m_frame_size, 0, 0, buf.GetNodeSize(), 0, GetNodeSize());
        }
        return dst;
    }

    // bit <-> fp32 with the values of the reference's CPU branch ((float)bit, i.e. 0 / 1; fp32 -> bit by > 0.5 as everywhere on this path)
    FrameBuffer ConvertTo(int data_type) const
    {
        if (data_type == m_type) return Clone();
        FrameBuffer dst(m_frame_size, m_shape, data_type);
        if (m_type == BB_TYPE_BIT && data_type == BB_TYPE_FP32 && m_mem->IsDeviceCurrent() && Manager::IsDeviceAvailable()) {
            BBCU_CHECK(bbcu_fp32_ConvBitToReal(static_cast<int const *>(m_mem->DevConst()), static_cast<float *>(dst.m_mem->Dev(true)), 0.0f, 1.0f,
                                               (int)GetNodeSize(), (int)m_frame_size, (int)(m_frame_stride / 4), (int)(dst.m_frame_stride / 4),
                                               Manager::Stream()));
            return dst;
        }
        dst.FillZero();
        for (index_t n = 0; n < GetNodeSize(); ++n)
            for (index_t f = 0; f < m_frame_size; ++f) dst.SetFP32(f, n, GetFP32(f, n));
        return dst;
    }

    // element access on the host mirror (slow path, as in the reference: FrameBuffer.h:1077-1146)
    float GetFP32(index_t frame, index_t node) const
    {
        auto base = static_cast<std::uint8_t const *>(m_mem->HostConst()) + node * m_frame_stride;
        if (m_type == BB_TYPE_FP32) return reinterpret_cast<float const *>(base)[frame];
        return (float)((reinterpret_cast<std::uint32_t const *>(base)[frame >> 5] >> (frame & 31)) & 1u);
    }
    void SetFP32(index_t frame, index_t node, float v)
    {
        auto base = static_cast<std::uint8_t *>(m_mem->Host()) + node * m_frame_stride;
        if (m_type == BB_TYPE_FP32) { reinterpret_cast<float *>(base)[frame] = v; return; }
        auto &w = reinterpret_cast<std::uint32_t *>(base)[frame >> 5];
        std::uint32_t m = 1u << (frame & 31);
        if (v > 0.5f) w |= m; else w &= ~m;            // include/bb/DataType.h:612-647, LSB first
    }

    // dense [frame][node] host array -> buffer (what FromNumpy receives from Python: frames on axis 0)
    void SetFrameMajor(float const *src)
    {
        index_t nodes = GetNodeSize();
        auto base = static_cast<std::uint8_t *>(m_mem->Host(true));
        std::memset(base, 0, m_mem->GetSize());
        for (index_t n = 0; n < nodes; ++n) {
            auto row = base + n * m_frame_stride;
            if (m_type == BB_TYPE_FP32) {
                for (index_t f = 0; f < m_frame_size; ++f) reinterpret_cast<float *>(row)[f] = src[f * nodes + n];
            } else {
                for (index_t f = 0; f < m_frame_size; ++f)
                    if (src[f * nodes + n] > 0.5f) reinterpret_cast<std::uint32_t *>(row)[f >> 5] |= 1u << (f & 31);
            }
        }
    }
    void GetFrameMajor(float *dst) const
    {
        index_t nodes = GetNodeSize();
        auto base = static_cast<std::uint8_t const *>(m_mem->HostConst());
        for (index_t n = 0; n < nodes; ++n) {
            auto row = base + n * m_frame_stride;
            if (m_type == BB_TYPE_FP32) {
                for (index_t f = 0; f < m_frame_size; ++f) dst[f * nodes + n] = reinterpret_cast<float const *>(row)[f];
            } else {
                for (index_t f = 0; f < m_frame_size; ++f)
                    dst[f * nodes + n] = (float)((reinterpret_cast<std::uint32_t const *>(row)[f >> 5] >> (f & 31)) & 1u);
            }
        }
    }
};

}   // namespace bb
