// SwiGLU, the gate of the feed-forward block between the gate+up projection and the down projection:
//   h[m][f] = silu(gu[m][f]) * gu[m][F + f],   silu(g) = g / (1 + exp(-g)),   gu = [gate | up], 2F wide.
// One definition in fp32 (correctly rounded division, expf, one multiplication), used by the stand-alone kernel and by
// every kernel that fuses it into its input stage, so that fused and unfused paths give the same bits.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace mpq {

__device__ __forceinline__ float swiglu_f32(float g, float u) { return __fdiv_rn(g, 1.0f + expf(-g)) * u; }

__device__ __forceinline__ float4 swiglu_f32x4(float4 g, float4 u)
{
    return make_float4(swiglu_f32(g.x, u.x), swiglu_f32(g.y, u.y), swiglu_f32(g.z, u.z), swiglu_f32(g.w, u.w));
}

}  // namespace mpq
