// Error-handling macros with the names and behaviour of the InferSpore sources
// (reference: src/utils/macro.h): CHECK prints and exits on a CUDA error,
// LLM_CHECK / LLM_CHECK_WITH_INFO throw std::runtime_error.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>

#ifndef CHECK
#define CHECK(call)                                                                     \
    do {                                                                                \
        const cudaError_t ispore_check_status_ = (call);                                \
        if (ispore_check_status_ != cudaSuccess) {                                      \
            std::printf("CUDA Error:\n    File:       %s\n    Line:       %d\n", __FILE__, __LINE__); \
            std::printf("    Error code: %d\n    Error text: %s\n", (int)ispore_check_status_,        \
                        cudaGetErrorString(ispore_check_status_));                      \
            std::exit(1);                                                               \
        }                                                                               \
    } while (0)
#endif

[[noreturn]] inline void throwRuntimeError(const char* const file, int const line,
                                           std::string const& info = "") {
    throw std::runtime_error(std::string("[oneLLM][ERROR] ") + info + " Assertion fail: " + file + ":" +
                             std::to_string(line) + " \n");
}

inline void llmAssert(bool result, const char* const file, int const line, std::string const& info = "") {
    if (!result) throwRuntimeError(file, line, info);
}

#define LLM_CHECK(val) llmAssert((val), __FILE__, __LINE__)
#define LLM_CHECK_WITH_INFO(val, info)                                   \
    do {                                                                 \
        const bool ispore_llm_ok_ = (val);                               \
        if (!ispore_llm_ok_) llmAssert(ispore_llm_ok_, __FILE__, __LINE__, (info)); \
    } while (0)

// cudaDeviceSynchronize + cudaGetLastError, throwing on failure.
inline void syncAndCheck(const char* const file, int const line) {
    cudaDeviceSynchronize();
    const cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess)
        throw std::runtime_error(std::string("[TM][ERROR] CUDA runtime error: ") + cudaGetErrorString(status) +
                                 " " + file + ":" + std::to_string(line) + " \n");
}
#define DeviceSyncAndCheckCudaError() syncAndCheck(__FILE__, __LINE__)
