// placeholder until the tcgen05 kernels land
#pragma once
#include "common.cuh"
namespace slime {
struct Bf16Plan { int tiles_x = 1, k1_tiles = 1, k2_tiles = 1; };
inline void bf16_plan(Bf16Plan&, const Geom&) {}
inline int bf16_setup(Bf16Plan&, const __nv_bfloat16*, const __nv_bfloat16*, int) { return -1; }
inline const char* bf16_error() { return "bf16 path not built"; }
inline int bf16_k1(Bf16Plan&, const __nv_bfloat16*, const float*, const float*, __nv_bfloat16*, __nv_bfloat16*, int*,
                   const Geom&, cudaStream_t) { return -1; }
inline int bf16_k2(Bf16Plan&, __nv_bfloat16*, const float*, const __nv_bfloat16*, const __nv_bfloat16*, float*,
                   __nv_bfloat16*, int*, const Geom&, cudaStream_t) { return -1; }
}
