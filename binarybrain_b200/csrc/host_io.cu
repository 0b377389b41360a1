// BinaryLut6 forward on HOST frame buffers: the call a host-resident caller makes (x and y live in host memory, as
// BinaryBrain's FrameBuffer does before its first device lock, include/bb/Memory.h:524-662).  The frame axis is cut
// into chunks of 4096 words; three stream-ordered slots each run  H2D copy -> kernel -> D2H copy  on their own stream,
// so the upload of chunk k+1, the kernel of chunk k and the download of chunk k-1 overlap and the PCIe link is busy in
// both directions at once.  With pinned host memory the whole call costs about max(upload, download) instead of
// their sum plus the kernel.  Device chunk buffers come from the device heap and are cached between calls.
#include <mutex>

#include "common.cuh"

namespace {

constexpr int kSlots      = 3;
constexpr int kChunkWords = 4096;     // 16 KiB per row and chunk; a multiple of the kernels' 256-word tile

struct HostIo {
    cudaStream_t stream[kSlots] = {};
    void *x[kSlots] = {}, *y[kSlots] = {};
    size_t x_bytes = 0, y_bytes = 0;
    void *idx = nullptr, *table = nullptr;
    size_t idx_bytes = 0, table_bytes = 0;
    bool ready = false;
};

std::mutex g_mu;
HostIo g_io[64];

int ensure(HostIo &io, size_t xb, size_t yb, size_t ib, size_t tb)
{
    if (!io.ready) {
        for (int s = 0; s < kSlots; ++s) BB200_CUDA(cudaStreamCreateWithFlags(&io.stream[s], cudaStreamNonBlocking));
        io.ready = true;
    }
    auto grow = [](void *&p, size_t &have, size_t want) -> int {
        if (have >= want) return 0;
        if (p) bbcu_LocalHeap_Free(p);
        p = bbcu_LocalHeap_Malloc(want);
        have = p ? want : 0;
        return p ? 0 : BBCU_ERR_NO_MEMORY;
    };
    if (io.x_bytes < xb) {
        for (int s = 0; s < kSlots; ++s) { size_t h = io.x_bytes; int rc = grow(io.x[s], h, xb); if (rc) return rc; }
        io.x_bytes = xb;
    }
    if (io.y_bytes < yb) {
        for (int s = 0; s < kSlots; ++s) { size_t h = io.y_bytes; int rc = grow(io.y[s], h, yb); if (rc) return rc; }
        io.y_bytes = yb;
    }
    int rc = grow(io.idx, io.idx_bytes, ib);
    if (rc) return rc;
    return grow(io.table, io.table_bytes, tb);
}

}   // namespace

extern "C" int bbcu_host_bit_BinaryLut6_Forward(const int *host_x_buf, int *host_y_buf, const int *host_input_index, const int *host_table,
                                                int input_node_size, int node_size, int frame_size, int frame_stride)
{
    BB200_REQUIRE_PTR(host_x_buf); BB200_REQUIRE_PTR(host_y_buf); BB200_REQUIRE_PTR(host_input_index); BB200_REQUIRE_PTR(host_table);
    BB200_REQUIRE(input_node_size > 0 && node_size >= 0 && frame_size >= 0, BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE((long long)frame_stride * 32 >= frame_size, BBCU_ERR_BAD_STRIDE);
    if (node_size == 0 || frame_size == 0) return BBCU_OK;
    const int dev = bbcu_GetDevice();
    BB200_REQUIRE(dev >= 0 && dev < 64, BBCU_ERR_NO_DEVICE);

    std::lock_guard<std::mutex> lock(g_mu);          // one host-buffer call per process at a time: the slots are shared
    HostIo &io = g_io[dev];
    const int words = (frame_size + 31) / 32;
    const int cw = words < kChunkWords ? ((words + 7) & ~7) : kChunkWords;       // device row stride of a chunk (32-byte rows)
    int rc = ensure(io, sizeof(int) * (size_t)input_node_size * cw, sizeof(int) * (size_t)node_size * cw,
                    sizeof(int) * 6 * (size_t)node_size, sizeof(int) * 2 * (size_t)node_size);
    if (rc) return rc;
    BB200_CUDA(cudaMemcpyAsync(io.idx, host_input_index, sizeof(int) * 6 * (size_t)node_size, cudaMemcpyHostToDevice, io.stream[0]));
    BB200_CUDA(cudaMemcpyAsync(io.table, host_table, sizeof(int) * 2 * (size_t)node_size, cudaMemcpyHostToDevice, io.stream[0]));
    BB200_CUDA(cudaStreamSynchronize(io.stream[0]));

    // On any error the copies already enqueued into the caller's host_y_buf are drained before the status goes back: the caller
    // may free or reuse its buffers as soon as this function returns.
    auto drain = [&](int status) {
        for (int s = 0; s < kSlots; ++s)
            if (cudaStreamSynchronize(io.stream[s]) != cudaSuccess) cudaGetLastError();
        return status;
    };
    const int chunks = (words + cw - 1) / cw;
    for (int k = 0; k < chunks; ++k) {
        const int s = k % kSlots;
        cudaStream_t st = io.stream[s];
        const int w0 = k * cw;
        const int nw = words - w0 < cw ? words - w0 : cw;
        const int frames_k = (k == chunks - 1) ? frame_size - w0 * 32 : nw * 32;
        cudaError_t e = cudaMemcpy2DAsync(io.x[s], sizeof(int) * (size_t)cw, host_x_buf + w0, sizeof(int) * (size_t)frame_stride, sizeof(int) * (size_t)nw,
                                          (size_t)input_node_size, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) { cudaGetLastError(); return drain((int)e); }
        rc = bbcu_bit_BinaryLut6_Forward(static_cast<const int *>(io.x[s]), static_cast<int *>(io.y[s]), static_cast<const int *>(io.idx),
                                         static_cast<const int *>(io.table), node_size, frames_k, cw, st);
        if (rc) return drain(rc);
        e = cudaMemcpy2DAsync(host_y_buf + w0, sizeof(int) * (size_t)frame_stride, io.y[s], sizeof(int) * (size_t)cw, sizeof(int) * (size_t)nw,
                              (size_t)node_size, cudaMemcpyDeviceToHost, st);
        if (e != cudaSuccess) { cudaGetLastError(); return drain((int)e); }
    }
    for (int s = 0; s < kSlots; ++s) {
        const cudaError_t e = cudaStreamSynchronize(io.stream[s]);
        if (e != cudaSuccess) { cudaGetLastError(); return drain((int)e); }
    }
    return BBCU_OK;
}

// Page-locked host memory for the buffers handed to the call above (pageable memory works too, but its copies are
// staged by the driver and do not overlap).
extern "C" void *bbcu_b200_host_alloc(size_t bytes)
{
    void *p = nullptr;
    if (cudaMallocHost(&p, bytes) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return p;
}

extern "C" void bbcu_b200_host_free(void *p)
{
    if (p && cudaFreeHost(p) != cudaSuccess) cudaGetLastError();
}
