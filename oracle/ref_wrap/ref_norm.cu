// TEST INFRASTRUCTURE.  Compiles the reference's own unit test
// tests/unittests/test_fused_addresidual_norm.cu from where it lies (its main()
// renamed) and exports its CPU function CPUfusedresidandRMSNorm (:33-55; only
// meaningful for rows of identical elements, see :39-46) and the reference's
// fp32 GPU launcher (src/kernels/fused_addresidual_norm.cu:143-170).  The fp16
// launcher is not exported: at hidden 4096 it asks for 2048 threads per block
// (:155-158) and its kernel reads through uninitialised pointers (:116-121).
#define main ref_test_fused_addresidual_norm_main
#include "tests/unittests/test_fused_addresidual_norm.cu"
#undef main

extern "C" {
__attribute__((visibility("default"))) void ref_cpu_fused_resid_rmsnorm_f32(float* residual, float* decoder_out,
                                                                           float* bias, float* scale, float eps,
                                                                           int hidden, int tokens) {
    CPUfusedresidandRMSNorm(residual, decoder_out, bias, scale, eps, hidden, tokens);
}
// hidden must be a multiple of 128 and at most 4096 so the reference's
// hidden/4-thread blocks are whole warps within the 1024-thread limit.
__attribute__((visibility("default"))) int ref_gpu_fused_resid_rmsnorm_f32(float* d_residual, float* d_decoder_out,
                                                                          float* d_bias, float* d_scale, float eps,
                                                                          int tokens, int hidden) {
    if (hidden % 128 != 0 || hidden > 4096 || hidden <= 0) return -1;
    TensorWrapper<float> res(GPU, FP32, {tokens, hidden}, d_residual), out(GPU, FP32, {tokens, hidden}, d_decoder_out);
    BaseWeight<float> norm;
    norm.bias = d_bias;
    launchFusedAddBiasResidualRMSNorm(&res, &out, norm, d_scale, eps);
    return 0;
}
}
