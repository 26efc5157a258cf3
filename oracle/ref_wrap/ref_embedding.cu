// TEST INFRASTRUCTURE.  Compiles the reference's own unit test
// tests/unittests/test_input_embedding.cu from where it lies (its main()
// renamed) and exports its CPU function cpuEmbedding (:35-41) and the
// reference's GPU launcher launchInputEmbedding (src/kernels/input_embedding.cu:25-45).
#define main ref_test_input_embedding_main
#include "tests/unittests/test_input_embedding.cu"
#undef main

extern "C" {
__attribute__((visibility("default"))) void ref_cpu_embedding_f32(const int* ids, float* output, float* table,
                                                                  int tokens, int hidden, int vocab) {
    cpuEmbedding(ids, output, table, tokens, hidden, vocab);
}
__attribute__((visibility("default"))) void ref_gpu_embedding_f32(int* d_ids, float* d_output, float* d_table,
                                                                  int tokens, int hidden) {
    TensorWrapper<int> ids(GPU, INT32, {tokens}, d_ids);
    TensorWrapper<float> out(GPU, FP32, {tokens, hidden}, d_output);
    EmbeddingWeight<float> table;
    table.data = d_table;
    launchInputEmbedding(&ids, &out, &table);
}
__attribute__((visibility("default"))) void ref_gpu_embedding_f16(int* d_ids, void* d_output, void* d_table,
                                                                  int tokens, int hidden) {
    TensorWrapper<int> ids(GPU, INT32, {tokens}, d_ids);
    TensorWrapper<half> out(GPU, FP16, {tokens, hidden}, static_cast<half*>(d_output));
    EmbeddingWeight<half> table;
    table.data = static_cast<half*>(d_table);
    launchInputEmbedding(&ids, &out, &table);
}
}
