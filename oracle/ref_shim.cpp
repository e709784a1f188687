// TEST INFRASTRUCTURE — not part of the shipped library.
//
// Binding shim for the reference's CPU-backend kernels. The reference's own
// csrc/cpu/pybind.cpp does not compile (it includes the CUDA-side headers whose
// signatures differ from the CPU definitions), so this translation unit
// forward-declares the entry points with the signatures their CPU
// definitions actually have (GLakeServe/csrc/cpu/attention.cpp:415-422 and
// :730-738, GLakeServe/csrc/cpu/cache.cpp:103-106,
// GLakeServe/csrc/cpu/pos_encoding.cpp:169-171,
// GLakeServe/csrc/cpu/layernorm.cpp:90-91, :104-105) and exposes them to Python.
// The reference sources themselves are compiled unmodified, from where they
// lie, by oracle/build_ref.py.
#include <torch/extension.h>

void paged_attention_v1(torch::Tensor &out, torch::Tensor &query,
                        torch::Tensor &key_cache, torch::Tensor &value_cache,
                        int num_kv_heads, float scale,
                        torch::Tensor &block_tables, torch::Tensor &seq_lens,
                        int block_size, int max_seq_len,
                        const c10::optional<torch::Tensor> &alibi_slopes,
                        const std::string &kv_cache_dtype, float kv_scale);

void paged_attention_v2(torch::Tensor &out, torch::Tensor &exp_sums,
                        torch::Tensor &max_logits, torch::Tensor &tmp_out,
                        torch::Tensor &query, torch::Tensor &key_cache,
                        torch::Tensor &value_cache, int num_kv_heads,
                        float scale, torch::Tensor &block_tables,
                        torch::Tensor &seq_lens, int block_size,
                        int max_seq_len,
                        const c10::optional<torch::Tensor> &alibi_slopes,
                        const std::string &kv_cache_dtype, float kv_scale);

void reshape_and_cache(torch::Tensor &key, torch::Tensor &value,
                       torch::Tensor &key_cache, torch::Tensor &value_cache,
                       torch::Tensor &slot_mapping,
                       const std::string &kv_cache_dtype, float kv_scale);

void rotary_embedding(torch::Tensor &positions, torch::Tensor &query,
                      torch::Tensor &key, int head_size,
                      torch::Tensor &cos_sin_cache, bool is_neox);

void rms_norm(torch::Tensor &out, torch::Tensor &input, torch::Tensor &weight,
              float epsilon);

void fused_add_rms_norm(torch::Tensor &input, torch::Tensor &residual,
                        torch::Tensor &weight, float epsilon);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("paged_attention_v1", &paged_attention_v1);
  m.def("paged_attention_v2", &paged_attention_v2);
  m.def("reshape_and_cache", &reshape_and_cache);
  m.def("rotary_embedding", &rotary_embedding);
  m.def("rms_norm", &rms_norm);
  m.def("fused_add_rms_norm", &fused_add_rms_norm);
}
