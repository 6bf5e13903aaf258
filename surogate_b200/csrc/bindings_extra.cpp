// Bindings for attention, MoE, NVFP4 and peer-memory communication kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "ext_api.h"

void sg_register_extra(pybind11::module_& m) { (void)m; }
