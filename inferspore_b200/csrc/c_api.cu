// Library-level entry points of the C ABI: error text, the thread-local stream
// used by the C++ launch templates, and the per-device status word that kernels
// set instead of trapping on bad data.
#include <stdarg.h>
#include <stdio.h>

#include <mutex>

#include "common.cuh"

namespace ispore {
namespace {

thread_local char g_error[512] = "";
thread_local cudaStream_t g_stream = nullptr;
thread_local bool g_programmatic_launch = false;

// One status word per device, in that device's memory.
__device__ unsigned g_device_status = 0;

constexpr int kMaxDevices = 64;
unsigned* g_status_addr[kMaxDevices] = {};
std::mutex g_status_mutex;

}  // namespace

bool programmatic_launch_enabled() { return g_programmatic_launch; }

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int check_launch(const char* what) {
    const cudaError_t e = cudaPeekAtLastError();
    if (e == cudaSuccess) return ISPORE_OK;
    (void)cudaGetLastError();  // clear a (non-sticky) launch-configuration error
    return fail(ISPORE_ELAUNCH, "%s: %s", what, cudaGetErrorString(e));
}

unsigned* device_status_ptr() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (g_status_addr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        g_status_addr[dev] = static_cast<unsigned*>(p);
    }
    return g_status_addr[dev];
}

#ifdef ISPORE_TUNING
static int g_tune[kTuneKeys] = {-1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1};
int tune(int key, int dflt) { return (key >= 0 && key < kTuneKeys && g_tune[key] >= 0) ? g_tune[key] : dflt; }
#endif

int sm_count() {
    static int cached[kMaxDevices] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return kNumSMs;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = kNumSMs;
        cached[dev] = n;
    }
    return cached[dev];
}

int resident_ctas(const void* kernel, int threads, size_t dynamic_smem) {
    // Fixed-size cache (no heap): (kernel, threads, smem) -> resident CTAs, per device.
    struct Entry {
        const void* kernel;
        int threads;
        size_t smem;
        int total;
    };
    constexpr int kSlots = 128;
    static std::mutex mutex;
    static Entry cache[kMaxDevices][kSlots] = {};
    static int used[kMaxDevices] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return kNumSMs;
    std::lock_guard<std::mutex> lock(mutex);
    for (int i = 0; i < used[dev]; ++i) {
        const Entry& e = cache[dev][i];
        if (e.kernel == kernel && e.threads == threads && e.smem == dynamic_smem) return e.total;
    }
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, dynamic_smem) != cudaSuccess ||
        per_sm <= 0) {
        (void)cudaGetLastError();
        per_sm = 1;
    }
    const int total = per_sm * sm_count();
    if (used[dev] < kSlots) cache[dev][used[dev]++] = Entry{kernel, threads, dynamic_smem, total};
    return total;
}

bool allow_dynamic_smem(const void* kernel, size_t bytes) {
    if (bytes <= 40 * 1024) return true;  // static shared memory of the kernel (a few KB) counts against the 48 KB default
    struct Entry {
        const void* kernel;
        size_t granted;
    };
    constexpr int kSlots = 128;
    static std::mutex mutex;
    static Entry cache[kMaxDevices][kSlots] = {};
    static int used[kMaxDevices] = {};
    int dev = 0;
    const bool cacheable = cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices;
    std::lock_guard<std::mutex> lock(mutex);
    Entry* slot = nullptr;
    if (cacheable) {
        for (int i = 0; i < used[dev]; ++i)
            if (cache[dev][i].kernel == kernel) slot = &cache[dev][i];
        if (slot != nullptr && slot->granted >= bytes) return true;
    }
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    if (cacheable) {
        if (slot == nullptr && used[dev] < kSlots) {
            slot = &cache[dev][used[dev]++];
            slot->kernel = kernel;
            slot->granted = 0;
        }
        if (slot != nullptr) slot->granted = bytes;
    }
    return true;
}

}  // namespace ispore

extern "C" {

#ifdef ISPORE_TUNING
__attribute__((visibility("default"))) void ispore_tune(int key, int value) {
    if (key >= 0 && key < ispore::kTuneKeys) ispore::g_tune[key] = value;
}
#endif

int ispore_version(void) { return 100; /* 0.1.0 */ }

const char* ispore_last_error_string(void) { return ispore::g_error; }

void ispore_set_stream(ispore_stream_t stream) { ispore::g_stream = static_cast<cudaStream_t>(stream); }

ispore_stream_t ispore_get_stream(void) { return ispore::g_stream; }

void ispore_set_programmatic_launch(int enable) { ispore::g_programmatic_launch = enable != 0; }

int ispore_get_programmatic_launch(void) { return ispore::g_programmatic_launch ? 1 : 0; }

int ispore_device_status(unsigned* flags_out, int clear) {
    if (flags_out == nullptr) return ispore::fail(ISPORE_ENULL, "device_status: flags_out is NULL");
    unsigned* p = ispore::device_status_ptr();
    if (p == nullptr) return ispore::fail(ISPORE_ELAUNCH, "device_status: no CUDA device");
    cudaError_t e = cudaMemcpy(flags_out, p, sizeof(unsigned), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && clear) e = cudaMemset(p, 0, sizeof(unsigned));
    if (e != cudaSuccess) return ispore::fail(ISPORE_ELAUNCH, "device_status: %s", cudaGetErrorString(e));
    return ISPORE_OK;
}

}  // extern "C"
