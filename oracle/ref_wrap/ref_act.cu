// TEST INFRASTRUCTURE.  Compiles the reference's own unit test
// tests/unittests/test_act.cu from where it lies (its main() renamed) and
// exports its CPU function CPUSwiGLU (test_act.cu:13-25) and the reference's
// GPU launcher launchAct (src/kernels/act_kernel.cu:57-71) through a C ABI, so
// the checker can run the unmodified reference code.
#define main ref_test_act_main
#include "tests/unittests/test_act.cu"
#undef main

extern "C" {
__attribute__((visibility("default"))) void ref_cpu_swiglu_f32(float* input, float* output, int rows, int inter) {
    CPUSwiGLU<float>(input, output, rows, inter);
}
__attribute__((visibility("default"))) void ref_cpu_swiglu_f16(void* input, void* output, int rows, int inter) {
    CPUSwiGLU<half>(static_cast<half*>(input), static_cast<half*>(output), rows, inter);
}
// Device pointers; default stream; asynchronous like the reference launcher.
__attribute__((visibility("default"))) void ref_gpu_act_f32(float* d_input, float* d_output, int rows, int inter) {
    TensorWrapper<float> in(GPU, FP32, {rows, 2, inter}, d_input), out(GPU, FP32, {rows, inter}, d_output);
    launchAct(&in, &out);
}
__attribute__((visibility("default"))) void ref_gpu_act_f16(void* d_input, void* d_output, int rows, int inter) {
    TensorWrapper<half> in(GPU, FP16, {rows, 2, inter}, static_cast<half*>(d_input)),
        out(GPU, FP16, {rows, inter}, static_cast<half*>(d_output));
    launchAct(&in, &out);
}
}
