// placeholder
#pragma once
#include "attn_simt.cuh"
namespace ggr {
struct MmaPlan { size_t smem; int ctas_per_sm; int min_keys; };
inline bool mma_decode_supported(int, int) { return false; }
inline MmaPlan mma_plan(int, int) { return MmaPlan{0, 1, 128}; }
inline int launch_mma_decode(const AttnArgs&, dim3, size_t, int, int, cudaStream_t) { return (int)cudaErrorNotSupported; }
}
