// DifferentiableLut6 training forward for callers that must not allocate device memory.
//
// bbcu_fp32_DifferentiableLut6_ForwardTraining keeps its per-node fp64 sums (sum y, sum y^2) in scratch
// memory that it takes from the device heap, i.e. from cudaMalloc, the first time a stream needs it or
// needs more of it.  Some callers cannot have that happen inside the call: code running under a memory
// budget that was handed out up front (an inference server or a training job that pre-plans all device
// memory and treats any later cudaMalloc as a bug), and code on a latency-critical path where the implicit
// device synchronisation of cudaMalloc / cudaFree is not acceptable.  The entry point below does the same
// computation with the sums in a fixed array that is part of this library's device image.
//
// Cost and limits: the array holds 2 x 65536 doubles = 1 MiB and every GPU that loads the library carries
// it until the process exits.  Layers with more than 65536 output nodes are rejected.  All calls on one
// device share the one array, so two calls whose GPU work can overlap (different streams, or different
// host threads on different streams) race on it; serialise them on one stream.
#include <mutex>

#include "common.cuh"

namespace {

constexpr int kNoAllocMaxNodes = 65536;

// File-scope device array.  In HOST code this name is only a handle for the runtime's symbol table -- it is
// not a device address and must never be handed to a kernel; the address comes from cudaGetSymbolAddress.
static __device__ __align__(256) double g_no_alloc_sums[2 * kNoAllocMaxNodes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
double *g_sums_addr[kMaxDevices] = {};

// Once per device, with that device current: resolve the array's device address.
int resolve_sums(double **out)
{
    int dev = -1;
    BB200_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return BBCU_ERR_NO_DEVICE;
    std::lock_guard<std::mutex> lock(g_setup_mu);
    if (g_sums_addr[dev] == nullptr) {
        void *p = nullptr;
        BB200_CUDA(cudaGetSymbolAddress(&p, g_no_alloc_sums));
        if (p == nullptr) return BBCU_ERR_NO_DEVICE;
        g_sums_addr[dev] = static_cast<double *>(p);
    }
    *out = g_sums_addr[dev];
    return BBCU_OK;
}

}   // namespace

extern "C" int bbcu_fp32_DifferentiableLut6_ForwardTraining_NoAlloc_MaxNodes(void) { return kNoAllocMaxNodes; }

// Same arguments, results and stream semantics as bbcu_fp32_DifferentiableLut6_ForwardTraining, but calls no
// cudaMalloc / cudaFree and no allocating library routine.  The first call on each device looks up the
// scratch array's address (cudaGetSymbolAddress); make that first call outside of any stream capture.
// The sums are cleared on the stream at the start of every call, so nothing of an earlier call leaks in.
extern "C" int bbcu_fp32_DifferentiableLut6_ForwardTraining_NoAlloc(const float *dev_x_buf, float *dev_y_buf, const int *dev_input_index,
                                                                    const float *dev_W, float *dev_mean_buf, float *dev_rstd_buf,
                                                                    float *dev_running_mean_buf, float *dev_running_var_buf, float gamma,
                                                                    float beta, float momentum, float unbinarize_bias, int node_size,
                                                                    int frame_size, int frame_stride, int lut_binarize, int binary_mode,
                                                                    bbcu_stream_t stream)
{
    BB200_REQUIRE_PTR(dev_mean_buf); BB200_REQUIRE_PTR(dev_rstd_buf); BB200_REQUIRE_PTR(dev_running_mean_buf); BB200_REQUIRE_PTR(dev_running_var_buf);
    BB200_REQUIRE(node_size >= 0 && (frame_size > 0 || node_size == 0), BBCU_ERR_BAD_SIZE);
    BB200_REQUIRE(node_size <= kNoAllocMaxNodes, BBCU_ERR_TOO_LARGE);      // more nodes than the fixed scratch array holds
    if (node_size == 0) return BBCU_OK;
    double *sums = nullptr;
    int rc = resolve_sums(&sums);
    if (rc) return rc;
    // pass 1 clears `sums` on the stream, stores the raw LUT values in y and accumulates the per-node sums;
    // pass 2 turns the sums into mean / rstd / running statistics and normalises y in place
    // (may_allocate = false: the kernel then converts each node's table itself instead of reading a converted copy from heap scratch)
    rc = bb200::dl6_forward_stats(dev_x_buf, dev_y_buf, dev_input_index, dev_W, sums, unbinarize_bias, node_size, frame_size, frame_stride,
                           lut_binarize, binary_mode, false, bb200::as_stream(stream));
    if (rc) return rc;
    return bbcu_fp32_DifferentiableLut6_ForwardNormalize(dev_y_buf, sums, dev_mean_buf, dev_rstd_buf, dev_running_mean_buf, dev_running_var_buf,
                                                         gamma, beta, momentum, node_size, frame_size, frame_stride, frame_size, binary_mode,
                                                         stream);
}
