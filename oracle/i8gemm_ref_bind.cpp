// Python binding for the reference's own dense W8A8 linear (csrc/i8gemm.cpp of the reference project,
// compiled where it lies, never copied).  On a non-Arm host that file builds its portable scalar path
// (backend "fallback").  Test infrastructure only: the oracle's restatement is checked against it.
#include <torch/extension.h>

#include <string>
#include <tuple>

std::tuple<at::Tensor, at::Tensor, int64_t, int64_t, int64_t, int64_t, std::string> i8gemm_prepare(
    at::Tensor weight, at::Tensor weight_scale, std::string backend);
void i8gemm_dynamic_scaled_mm(at::Tensor output, at::Tensor input, at::Tensor packed_weight, at::Tensor weight_scale,
                              c10::optional<at::Tensor> bias, int64_t K, int64_t N, int64_t Kp, int64_t Np,
                              int64_t nthreads);
void i8gemm_dynamic_scaled_mm_pair(at::Tensor first_output, at::Tensor second_output, at::Tensor input,
                                   at::Tensor first_packed_weight, at::Tensor first_weight_scale, int64_t K,
                                   int64_t first_N, int64_t Kp, int64_t first_Np, at::Tensor second_packed_weight,
                                   at::Tensor second_weight_scale, int64_t second_N, int64_t second_Np,
                                   int64_t nthreads);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("i8gemm_prepare", &i8gemm_prepare);
  m.def("i8gemm_dynamic_scaled_mm", &i8gemm_dynamic_scaled_mm);
  m.def("i8gemm_dynamic_scaled_mm_pair", &i8gemm_dynamic_scaled_mm_pair);
}
