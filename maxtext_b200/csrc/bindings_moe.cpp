// Bindings for the mixture-of-experts kernels (router top-k, permutation, grouped GEMM).
#include <torch/extension.h>

void register_moe(pybind11::module_& m) { (void)m; }
