// Bindings for the attention kernels (flash attention forward / backward).
#include <torch/extension.h>

void register_attention(pybind11::module_& m) { (void)m; }
