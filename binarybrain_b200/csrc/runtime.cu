// Device manager, caching device heap, per-stream scratch and launch heuristics.
//
// Replaces BinaryBrain's cuda/Manager.cu:15-55 (device select + host-only flag) and
// cuda/LocalHeap.cu:13-201 (caching allocator over cudaMalloc).  Differences by design:
//   - one pool per device and a mutex around it (the reference keeps one process-wide singleton
//     with no locking, cuda/LocalHeap.cu:172-201);
//   - free blocks are kept in a size-ordered multimap, so reuse is a lower_bound lookup instead of
//     a std::sort on every free (cuda/LocalHeap.cu:142-153);
//   - out of memory returns NULL after one garbage-collect-and-retry; nothing exits the process;
//   - freed blocks stay cached until they add up to half of the device's memory (the reference gives its cache back at 1.5x
//     the high-water mark, i.e. on nearly every step of a network with layers of different sizes);
//   - block sizes are rounded up to 512 bytes so that every row a caller carves out of a block
//     keeps the 256-byte alignment cudaMalloc gives.
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "async_copy.cuh"

namespace bb200 {

namespace {

struct Pool {
    std::mutex mu;
    std::unordered_map<void *, size_t> live;          // ptr -> block size
    std::multimap<size_t, void *> cached;             // block size -> ptr
    size_t live_bytes = 0, cached_bytes = 0, max_alloc = 0, byte_limit = 0;
    std::map<std::pair<cudaStream_t, int>, std::pair<void *, size_t>> scratch;     // (stream, slot) -> block
};

std::mutex g_pools_mu;
std::map<int, Pool *> g_pools;
bool g_host_only = false;
size_t g_byte_limit = 0;

Pool &pool_of_current_device()
{
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> g(g_pools_mu);
    auto it = g_pools.find(dev);
    if (it == g_pools.end()) it = g_pools.emplace(dev, new Pool()).first;
    return *it->second;
}

void release_cached_locked(Pool &p)
{
    for (auto &kv : p.cached) cudaFree(kv.second);
    p.cached.clear();
    p.cached_bytes = 0;
}

}   // namespace

const DeviceInfo &device_info()
{
    static std::mutex mu;
    static std::map<int, DeviceInfo> infos;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> g(mu);
    auto it = infos.find(dev);
    if (it == infos.end()) {
        DeviceInfo di{148, (size_t)126 << 20, (size_t)180 << 30};
        int v = 0;
        size_t free_b = 0, total_b = 0;
        if (cudaMemGetInfo(&free_b, &total_b) == cudaSuccess && total_b > 0) di.total_bytes = total_b; else cudaGetLastError();
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) di.sm_count = v;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, dev) == cudaSuccess && v > 0) di.l2_bytes = (size_t)v;
        it = infos.emplace(dev, di).first;
    }
    return it->second;
}

int frame_tile(long long rows_touched, int bits_per_row_frame, int node_groups, int frame_size, int max_tile)
{
    const DeviceInfo &di = device_info();
    // a fifth of L2 for the tile: both dies cache what they touch, and outputs stream through as well
    const double budget_bits = 8.0 * (double)di.l2_bytes / 5.0;
    double per_frame = (double)(rows_touched > 0 ? rows_touched : 1) * (double)bits_per_row_frame;
    long long t = (long long)(budget_bits / per_frame);
    t = (t / kFramesPerIterHost) * kFramesPerIterHost;
    if (t < kFramesPerIterHost) t = kFramesPerIterHost;
    if (t > max_tile) t = max_tile;
    // keep at least ~4 CTAs per SM in flight while the tile is still wider than one iteration
    const long long want_ctas = 4LL * di.sm_count;
    while (t > kFramesPerIterHost && (long long)node_groups * ((frame_size + t - 1) / t) < want_ctas) t -= kFramesPerIterHost;
    return (int)t;
}

// The fault word lives in the library's device image (zero until a kernel records a fault), so that no launch path ever has to
// allocate it: in host code the symbol below is only a handle, its device address is looked up once per device.
static __device__ __align__(256) int g_fault_word[64];

int *fault_word()
{
    static std::mutex mu;
    static std::map<int, int *> words;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> g(mu);
    auto it = words.find(dev);
    if (it == words.end()) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_fault_word) != cudaSuccess || p == nullptr) { cudaGetLastError(); return nullptr; }
        it = words.emplace(dev, static_cast<int *>(p)).first;
    }
    return it->second;
}

void *stream_scratch(cudaStream_t stream, size_t bytes, int slot)
{
    if (slot < 0 || slot >= kScratchSlots) return nullptr;
    const std::pair<cudaStream_t, int> key(stream, slot);
    if (bytes == 0) bytes = 256;
    Pool &p = pool_of_current_device();
    {
        std::lock_guard<std::mutex> g(p.mu);
        auto it = p.scratch.find(key);
        if (it != p.scratch.end() && it->second.second >= bytes) return it->second.first;
    }
    // grow: the old block goes back to the heap cache (work already enqueued on it is stream-ordered
    // before anything a later owner enqueues only if that owner uses the same stream, so hand it to
    // the heap only after the stream has drained)
    void *fresh = bbcu_LocalHeap_Malloc(bytes);
    if (!fresh) return nullptr;
    void *old = nullptr;
    {
        std::lock_guard<std::mutex> g(p.mu);
        auto it = p.scratch.find(key);
        if (it != p.scratch.end()) old = it->second.first;
        p.scratch[key] = std::make_pair(fresh, bytes);
    }
    if (old) {
        cudaStreamSynchronize(stream);
        bbcu_LocalHeap_Free(old);
    }
    return fresh;
}

}   // namespace bb200

using namespace bb200;

extern "C" const char *bbcu_b200_error_string(int status)
{
    switch (status) {
    case BBCU_OK:               return "ok";
    case BBCU_ERR_NULL_POINTER: return "bbcu_b200: a required pointer argument is NULL";
    case BBCU_ERR_BAD_SIZE:     return "bbcu_b200: a size argument is negative or inconsistent";
    case BBCU_ERR_BAD_STRIDE:   return "bbcu_b200: a stride is smaller than the frame count or a pointer is misaligned";
    case BBCU_ERR_NO_DEVICE:    return "bbcu_b200: no CUDA device available";
    case BBCU_ERR_NO_MEMORY:    return "bbcu_b200: device memory exhausted";
    case BBCU_ERR_TOO_LARGE:    return "bbcu_b200: problem size exceeds what this entry point supports";
    default: break;
    }
    if (status > 0) return cudaGetErrorString((cudaError_t)status);
    return "bbcu_b200: unknown status";
}

extern "C" int bbcu_b200_abi_version(void) { return 1; }

// Synchronises the device and returns the first fault code a kernel recorded (0 = none), clearing it.
extern "C" int bbcu_b200_device_fault(void)
{
    int v = 0;
    int *w = fault_word();
    if (w == nullptr || cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v != 0) cudaMemset(w, 0, sizeof(int));
    return v;
}

// Self-test of the bounded-wait path that the pipelined kernels share: one warp arms a barrier for 16 bytes that no copy will ever
// deliver, waits with a small attempt limit, gives up as a whole warp, records the fault code and returns.  Nothing hangs and
// nothing faults; afterwards bbcu_b200_device_fault() reports 1 once.
namespace bb200 {
__global__ void k_selftest_wait_expiry(int *fault, int attempts)
{
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_init_fence();
    }
    __syncwarp();
    if (threadIdx.x == 0) mbar_arrive_expect_tx(&bar, 16u);
    __syncwarp();
    bool ok = false;
    for (int i = 0; i < attempts && !ok; ++i) ok = mbar_try_wait(&bar, 0u);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok && threadIdx.x == 0) atomicCAS(fault, 0, kFaultBarrierTimeout);
}
}   // namespace bb200

extern "C" int bbcu_b200_selftest_wait_expiry(bbcu_stream_t stream)
{
    int *w = fault_word();
    if (w == nullptr) return BBCU_ERR_NO_DEVICE;
    k_selftest_wait_expiry<<<1, 32, 0, as_stream(stream)>>>(w, 2000);
    return launch_status();
}

// ---------------------------------------------------------------------------------------------- manager
extern "C" int bbcu_GetDeviceCount(void)
{
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

extern "C" int bbcu_GetDevice(void)
{
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess) { cudaGetLastError(); return -1; }
    return d;
}

extern "C" void bbcu_SetDevice(int device)
{
    if (cudaSetDevice(device) != cudaSuccess) cudaGetLastError();
}

extern "C" void bbcu_SetHostOnly(int host_only) { g_host_only = host_only != 0; }
extern "C" int  bbcu_IsHostOnly(void)           { return g_host_only ? 1 : 0; }
extern "C" int  bbcu_IsDeviceAvailable(void)    { return (!g_host_only && bbcu_GetDeviceCount() > 0) ? 1 : 0; }

// ---------------------------------------------------------------------------------------------- heap
extern "C" void bbcu_LocalHeap_SetByteLimit(size_t bytes)
{
    g_byte_limit = bytes;
}

extern "C" void *bbcu_LocalHeap_Malloc(size_t size)
{
    if (size == 0) size = 4;                                   // include/bbcu/bbcu_util.h:91
    size = (size + 511) & ~(size_t)511;
    Pool &p = pool_of_current_device();
    std::lock_guard<std::mutex> g(p.mu);

    // reuse a cached block of at least `size` and less than 1.5x of it (cuda/LocalHeap.cu:94)
    auto it = p.cached.lower_bound(size);
    if (it != p.cached.end() && it->first < size + size / 2 + 512) {
        void *ptr = it->second;
        size_t bs = it->first;
        p.cached.erase(it);
        p.cached_bytes -= bs;
        p.live.emplace(ptr, bs);
        p.live_bytes += bs;
        if (p.live_bytes > p.max_alloc) p.max_alloc = p.live_bytes;
        return ptr;
    }
    if (g_byte_limit && p.live_bytes + p.cached_bytes + size > g_byte_limit) release_cached_locked(p);
    if (g_byte_limit && p.live_bytes + size > g_byte_limit) return nullptr;
    // The reference trims its cache whenever live + cached passes 1.5x the high-water mark (cuda/LocalHeap.cu:115-117).  A network
    // whose layers have different buffer sizes crosses that mark every step, and each trim is a cudaFree per block (a device
    // synchronisation plus the unmapping: measured 100 ms per layer of a LUT-CNN forward, against 0.4 ms of kernels).  Here the
    // cache is only given back when it holds more than half of the device's memory, on a byte limit, or when cudaMalloc fails.
    if (p.cached_bytes > 0 && p.cached_bytes + size > device_info().total_bytes / 2) release_cached_locked(p);

    void *ptr = nullptr;
    cudaError_t e = cudaMalloc(&ptr, size);
    if (e != cudaSuccess) {
        cudaGetLastError();
        release_cached_locked(p);                              // cuda/LocalHeap.cu:120-130
        e = cudaMalloc(&ptr, size);
        if (e != cudaSuccess) { cudaGetLastError(); return nullptr; }
    }
    p.live.emplace(ptr, size);
    p.live_bytes += size;
    if (p.live_bytes > p.max_alloc) p.max_alloc = p.live_bytes;
    return ptr;
}

extern "C" void bbcu_LocalHeap_Free(void *ptr)
{
    if (!ptr) return;
    Pool &p = pool_of_current_device();
    std::lock_guard<std::mutex> g(p.mu);
    auto it = p.live.find(ptr);
    if (it == p.live.end()) return;                            // not ours (or another device's): ignore
    size_t bs = it->second;
    p.live.erase(it);
    p.live_bytes -= bs;
    p.cached.emplace(bs, ptr);
    p.cached_bytes += bs;
}

extern "C" size_t bbcu_LocalHeap_GetMaxAllocSize(void)
{
    Pool &p = pool_of_current_device();
    std::lock_guard<std::mutex> g(p.mu);
    return p.max_alloc;
}

extern "C" size_t bbcu_LocalHeap_GetAllocatedSize(void)
{
    Pool &p = pool_of_current_device();
    std::lock_guard<std::mutex> g(p.mu);
    return p.live_bytes;
}

extern "C" void bbcu_LocalHeap_GarbageCollect(void)
{
    Pool &p = pool_of_current_device();
    std::vector<void *> scratch;
    {
        std::lock_guard<std::mutex> g(p.mu);
        for (auto &kv : p.scratch) scratch.push_back(kv.second.first);
        p.scratch.clear();
    }
    if (!scratch.empty()) cudaDeviceSynchronize();
    for (void *s : scratch) bbcu_LocalHeap_Free(s);
    std::lock_guard<std::mutex> g(p.mu);
    release_cached_locked(p);
}
