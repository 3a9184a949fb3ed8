// Python binding for the reference's own CUDA append launcher, and nothing else.
//
// TEST INFRASTRUCTURE ONLY.  The reference binds six kernels in one module
// (csrc/src/bindings.cpp:43-49,74-75); the paged KV path needs one of them.  This file declares that
// launcher - it is defined in the reference's csrc/kernels/paged_kv_cache.cu, which the recipe in
// ref_cuda.py compiles where it lies in the reference checkout - and exposes it under the reference's
// name, so that the GPU tests can run the unmodified reference kernel beside libbarqkv.

#include <torch/extension.h>

void paged_kv_append_cuda(torch::Tensor key_cache, torch::Tensor value_cache, torch::Tensor seq_lens,
                          torch::Tensor key_states, torch::Tensor value_states);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("paged_kv_append_", &paged_kv_append_cuda, "the reference's paged KV append (CUDA)");
}
