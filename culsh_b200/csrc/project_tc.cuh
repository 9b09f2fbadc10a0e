// Tensor-core projection path (placeholder until the tcgen05 kernel lands).
#pragma once

#include "common.cuh"

namespace culsh_b200 {

inline void prepare_project_tc(const CtxPtr&, const float*, int, int, DevBuf<uint8_t>&) {}

inline bool launch_project_tc(const CtxPtr&, cudaStream_t, int, const float*, const float*,
                              const uint8_t*, const float*, int, int, int, int, const KeySpec&,
                              uint32_t*, uint8_t*, int, int) {
    return false;
}

}  // namespace culsh_b200
