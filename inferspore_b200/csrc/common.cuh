// Shared device/host helpers for the sm_100a layer kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ispore_kernels.h"

namespace ispore {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs (fallback when the device query fails)

// ---- host-side status plumbing (c_api.cu owns the storage) -------------------
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);
unsigned* device_status_ptr();  // address of the per-device status word (device memory)
int sm_count();                 // SMs of the current device (cached)
// CTAs of `kernel` that are resident at once on the whole current device for the
// given block size / dynamic shared memory (occupancy query, cached per kernel
// and device).  Persistent grid-stride kernels launch exactly this many CTAs:
// one more would wait for a free slot and start its whole share of the work late.
int resident_ctas(const void* kernel, int threads, size_t dynamic_smem);
// Makes sure `kernel` may be launched with `bytes` of dynamic shared memory on the current device.
// Sizes well inside the 48 KB default (40 KB, leaving room for the kernel's static shared memory)
// need nothing; above that cudaFuncSetAttribute is called once per
// (device, kernel) for the largest size seen so far, not on every launch.  Returns false when the
// runtime refuses (the sticky-free error is cleared).
bool allow_dynamic_smem(const void* kernel, size_t bytes);
template <typename Kernel>
inline bool allow_dynamic_smem(Kernel kernel, size_t bytes) {
    return allow_dynamic_smem(reinterpret_cast<const void*>(kernel), bytes);
}

// ---- programmatic dependent launch ---------------------------------------------
// A kernel launched through launch_chained() may be scheduled before its predecessor on the
// stream has fully retired (the launch carries cudaLaunchAttributeProgrammaticStreamSerialization
// when the calling thread has switched that on with ispore_set_programmatic_launch).  Every kernel
// launched this way starts with chain_begin(): it waits until the predecessor grid has completed
// and its memory is visible, before the first global access.  Launched without the attribute the
// instruction is a no-op, so the same kernel serves both modes.  The wait is unconditional and
// precedes every early return, so a grid can only complete after its predecessor has: ordering
// stays transitive along the stream.
// The successor is released when this grid's CTAs exit (no explicit early trigger).  Measured on
// B200 over the eight-kernel chain, CUDA-graph replay: an early trigger at the top of every kernel
// (griddepcontrol.launch_dependents, so that the successor's CTAs take their places during this
// kernel's last wave and wait there) made the chain 11-12 % SLOWER at 8,192 and at 65,536 tokens
// (390 -> 437 us, 2.91 -> 3.22 ms); without it the attribute is neutral inside a graph (390 us)
// and saves 5 % on launches issued one by one at the small size (411 -> 391 us).
bool programmatic_launch_enabled();  // thread-local, c_api.cu

#ifndef ISPORE_CHAIN_MODE
#define ISPORE_CHAIN_MODE 1  // experiments: 0 = also trigger the successor at the top of the kernel
#endif
__device__ __forceinline__ void chain_begin() {
    if (ISPORE_CHAIN_MODE == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (ISPORE_CHAIN_MODE != 2) asm volatile("griddepcontrol.wait;" ::: "memory");  // 2: nothing (measurement only)
}

template <typename... KArgs, typename... Args>
inline void launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t dynamic_smem, cudaStream_t st,
                           Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = dynamic_smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    if (programmatic_launch_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);  // the caller reads the status with check_launch()
}

// Launch-shape experiments: a build with -DISPORE_TUNING exports ispore_tune(key, value)
// and dispatchers consult tune(key, default); the shipped build compiles this to the default.
enum TuneKey { kTuneRmsnorm = 0, kTuneSoftmax, kTuneAct, kTuneEmbedding, kTuneQkv, kTuneConcat, kTuneTopk,
               kTuneMhaChunk, kTuneMhaCtasPerSm, kTuneMhaGroup, kTuneMhaStaged, kTuneKeys };
#ifdef ISPORE_TUNING
int tune(int key, int dflt);
#else
inline int tune(int, int dflt) { return dflt; }
#endif

template <typename Kernel>
inline int persistent_grid(Kernel kernel, int threads, size_t dynamic_smem, int64_t work_items, int waves = 1) {
    const int64_t cap = static_cast<int64_t>(waves) *
                        resident_ctas(reinterpret_cast<const void*>(kernel), threads, dynamic_smem);
    return static_cast<int>(work_items < cap ? (work_items > 0 ? work_items : 1) : cap);
}

// ---- storage-type traits ------------------------------------------------------
// One 128-bit vector holds 4 floats or 8 halves.
template <typename T>
struct VecTraits;
template <>
struct VecTraits<float> {
    static constexpr int kElems = 4;
};
template <>
struct VecTraits<__half> {
    static constexpr int kElems = 8;
};

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) {
    return v;
}
template <>
__device__ __forceinline__ float to_float<__half>(__half v) {
    return __half2float(v);
}
template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) {
    return v;
}
template <>
__device__ __forceinline__ __half from_float<__half>(float v) {
    return __float2half_rn(v);
}

// ---- 128-bit global accesses with cache policy ---------------------------------
// Activations are touched once: stream them (evict-first) so that small reused
// operands (gamma, bias, masks, frequency tables) keep their L2 lines.
__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }
__device__ __forceinline__ uint4 ld_keep(const uint4* p) { return __ldg(p); }
__device__ __forceinline__ void st_stream(uint4* p, uint4 v) { __stcs(p, v); }

// A 128-bit vector viewed as N fp32 lanes after widening (4 for float, 8 for half).
template <typename T>
struct Unpacked;
template <>
struct Unpacked<float> {
    float v[4];
};
template <>
struct Unpacked<__half> {
    float v[8];
};

__device__ __forceinline__ void unpack(const uint4& raw, Unpacked<float>& out) {
    out.v[0] = __uint_as_float(raw.x);
    out.v[1] = __uint_as_float(raw.y);
    out.v[2] = __uint_as_float(raw.z);
    out.v[3] = __uint_as_float(raw.w);
}
__device__ __forceinline__ void unpack(const uint4& raw, Unpacked<__half>& out) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
        float2 f = __half22float2(h);
        out.v[2 * i] = f.x;
        out.v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ uint4 pack(const Unpacked<float>& in) {
    return make_uint4(__float_as_uint(in.v[0]), __float_as_uint(in.v[1]), __float_as_uint(in.v[2]),
                      __float_as_uint(in.v[3]));
}
__device__ __forceinline__ uint4 pack(const Unpacked<__half>& in) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h = __floats2half2_rn(in.v[2 * i], in.v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// Rounds every lane to the storage type and back (identity for float).  Used
// where the reference stores an intermediate in the activation type.
__device__ __forceinline__ void round_to_storage(Unpacked<float>&) {}
__device__ __forceinline__ void round_to_storage(Unpacked<__half>& x) {
#pragma unroll
    for (int i = 0; i < 8; ++i) x.v[i] = __half2float(__float2half_rn(x.v[i]));
}

// ---- reductions -------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// 2^x through the SFU (ex2.approx, ~2^-22 relative error, denormals flushed).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace ispore
