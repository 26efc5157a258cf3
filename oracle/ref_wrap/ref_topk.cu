// TEST INFRASTRUCTURE.  Exports the reference's GPU top-K launcher
// (src/kernels/topK.cu:76-110, launchTopKforBeamSearch: K fixed at 5, 8 blocks
// per row, 256 threads) through a C ABI; the reference has no CPU function and
// no unit test for it.  The wrapper refuses everything outside the domain on
// which the two kernels are functional:
//  * one row only: round 2 reads topK_ids[i] where it means
//    topK_ids[data_offset] (.cu:64), the same address only for row 0, and the
//    launcher caps the grids at 1024 blocks, i.e. 128 rows (.cu:98-101);
//  * the data must be positive (the kernel is meant for probabilities): empty
//    list slots carry the value -1e-20 (topK.h:14-19) and are re-inserted by
//    the block reduction (.cu:9-15), so they outrank every negative element.
//    Positivity of the data is the caller's side of the contract; the wrapper
//    cannot see device data and only checks the shape.
// Scratch [1, 8, 5] ids and values are the caller's, as in the reference.
#include "src/kernels/topK.h"

extern "C" {
__attribute__((visibility("default"))) int ref_gpu_topk_k() { return 5; }
__attribute__((visibility("default"))) int ref_gpu_topk_blocks_per_row() { return 8; }

__attribute__((visibility("default"))) int ref_gpu_topk_f32(float* d_probs, int rows, int vocab, int* d_scratch_ids,
                                                           float* d_scratch_vals, int* d_final_ids,
                                                           float* d_final_vals) {
    if (rows != 1 || vocab < 1) return -1;
    TensorWrapper<float> probs(GPU, FP32, {rows, vocab}, d_probs);
    TensorWrapper<int> ids(GPU, INT32, {rows, 8, 5}, d_scratch_ids), fin_ids(GPU, INT32, {rows, 5}, d_final_ids);
    TensorWrapper<float> vals(GPU, FP32, {rows, 8, 5}, d_scratch_vals), fin_vals(GPU, FP32, {rows, 5}, d_final_vals);
    launchTopKforBeamSearch(&probs, &ids, &vals, &fin_ids, &fin_vals);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
__attribute__((visibility("default"))) int ref_gpu_topk_f16(void* d_probs, int rows, int vocab, int* d_scratch_ids,
                                                           void* d_scratch_vals, int* d_final_ids,
                                                           void* d_final_vals) {
    if (rows != 1 || vocab < 1) return -1;
    TensorWrapper<half> probs(GPU, FP16, {rows, vocab}, static_cast<half*>(d_probs));
    TensorWrapper<int> ids(GPU, INT32, {rows, 8, 5}, d_scratch_ids), fin_ids(GPU, INT32, {rows, 5}, d_final_ids);
    TensorWrapper<half> vals(GPU, FP16, {rows, 8, 5}, static_cast<half*>(d_scratch_vals)),
        fin_vals(GPU, FP16, {rows, 5}, static_cast<half*>(d_final_vals));
    launchTopKforBeamSearch(&probs, &ids, &vals, &fin_ids, &fin_vals);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
}
