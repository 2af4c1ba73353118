// Python binding of the REFERENCE's own scoreboard check, compiled from the reference checkout
// (src/psh/bucket_sanitizer_cpu.cpp:92-176) for pinning the library's f3d_batch_bucket_sanitizer_cpu and the oracle's
// scoreboard_check.  TEST INFRASTRUCTURE ONLY.  This file holds only the declaration and the binding, as
// src/f3d_frontend.cu:86-88,133 do; the function body is compiled from the reference's source file where it lies.
#include <torch/extension.h>

namespace f3d {
void batch_bucket_sanitizer_cpu(at::Tensor &bucket_id, at::Tensor &bucket_counter, at::Tensor &bucket_offset,
                                at::Tensor &offset_check_table, at::Tensor &bucket_residual, at::Tensor &batch_sep,
                                at::Tensor &offset_maxcnt, uint32_t batch_size, uint16_t num_bucket);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("batch_bucket_sanitizer_cpu", f3d::batch_bucket_sanitizer_cpu);
}
