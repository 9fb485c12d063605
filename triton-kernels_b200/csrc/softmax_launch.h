// Host-side declaration for the row softmax kernels.
#pragma once

#include <cuda_runtime.h>

#include "../../include/b200attn.h"

namespace b200attn {

int launch_softmax(const b200attn_softmax_args_t& a, int sm_count, cudaStream_t stream);

}  // namespace b200attn
