// Library-wide entry points of the C ABI and the per-device cache of the multiprocessor count.
#include "cam_common.cuh"

#include <map>
#include <mutex>
#include <tuple>

int cam_sm_count() {
    static int count[64] = {0};          // 0: not read yet (every thread that finds 0 reads the same attribute: no lock needed)
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int v = __atomic_load_n(&count[dev], __ATOMIC_RELAXED);
    if (v == 0) {
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v < 1) v = 148;
        __atomic_store_n(&count[dev], v, __ATOMIC_RELAXED);
    }
    return v;
}

// Resident blocks per multiprocessor of (kernel, block size, dynamic shared memory) on the current device. The occupancy query is a
// driver call, so its answers are kept: first in a few slots private to the calling thread (a launch loop asks the same few questions
// again and again: no lock, no tree walk on that path), behind them in a map shared by all threads.
int cam_blocks_per_sm(const void * kernel, int threads, size_t smem) {
    struct Slot { int dev; const void * kernel; int threads; size_t smem; int per_sm; };
    static thread_local Slot recent[8] = {};
    static thread_local unsigned next = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    for (const Slot & s : recent)
        if (s.kernel == kernel && s.dev == dev && s.threads == threads && s.smem == smem) return s.per_sm;
    static std::mutex mu;
    static std::map<std::tuple<int, const void *, int, size_t>, int> cache;
    const auto key = std::make_tuple(dev, kernel, threads, smem);
    int per_sm = 0;
    {
        std::lock_guard<std::mutex> lock(mu);
        const auto it = cache.find(key);
        if (it != cache.end()) per_sm = it->second;
    }
    if (per_sm == 0) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess || per_sm < 1) per_sm = 1;
        std::lock_guard<std::mutex> lock(mu);
        cache[key] = per_sm;
    }
    recent[next++ & 7u] = Slot{dev, kernel, threads, smem, per_sm};
    return per_sm;
}

// The ABI's version: bumped when an entry's parameters change.
extern "C" int cam_abi_version(void) { return 1; }

// Text of an entry's return value: 0 ok, negative = an argument refusal of this library, positive = a cudaError_t.
extern "C" const char * cam_error_string(int code) {
    switch (code) {
        case CAM_OK: return "ok";
        case CAM_ERR_ARG: return "invalid argument (a count, a size or a null pointer the entry does not take)";
        case CAM_ERR_ALIGN: return "a pointer or stride is not aligned for 128-bit access";
        case CAM_ERR_SHAPE: return "a row length, head layout or position range outside what the kernels are built for";
        case CAM_ERR_CAPACITY: return "more than a fixed-size buffer of the library holds";
        default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error";
    }
}
