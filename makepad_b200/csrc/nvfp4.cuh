// NVFP4 (e2m1 codes, e4m3 scale per 16, fp32 tensor scale): device types,
// exact export, scale-factor tiling and the block-scaled GEMM.
//
// No reference source exists for this path (the makepad/makepad snapshot has no
// quantised-linear code); the operator is specified by the task configuration.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/mpq.h"

namespace mpq {

struct Nvfp4Dev {
    int64_t N = 0, K = 0;
    float tensor_scale = 1.f;
    uint8_t* codes = nullptr;          // canonical [N][K/2]: already K-major, which is what the MMA wants
    uint8_t* sf_tiled = nullptr;       // scale factors in the 128x4 tile order the tensor core reads (the only copy)
    size_t sf_tiled_bytes = 0;
    size_t device_bytes() const { return (size_t)N * (K / 2) + sf_tiled_bytes; }
    void release()
    {
        cudaFree(codes); cudaFree(sf_tiled);
        codes = sf_tiled = nullptr;
    }
};

struct Nvfp4Scratch {
    uint8_t* sfa_tiled = nullptr;      // activation scale factors re-tiled per call
    size_t sfa_bytes = 0;
    int* status = nullptr;             // set non-zero when a bounded wait in the GEMM kernel ran out
    void release() { cudaFree(sfa_tiled); cudaFree(status); sfa_tiled = nullptr; status = nullptr; sfa_bytes = 0; }
};

void nvfp4_dequant_launch(const uint8_t* codes, const uint8_t* sf, float ts, int64_t R, int64_t K, float* out, cudaStream_t s);
int32_t nvfp4_weight_build(Nvfp4Dev& w, int64_t N, int64_t K, const uint8_t* codes_host, const uint8_t* sf_host, float ts,
                           int* launches, std::string& err);
// fp32 (or bf16) rows -> canonical NVFP4 codes [R][K/2] and e4m3 scales [R][K/16]
void nvfp4_quantize_launch(const void* x, bool bf16, bool swiglu, int64_t R, int64_t K, float ts, uint8_t* codes, uint8_t* sf, cudaStream_t s);
// bytes of a weight's tiled scale factors in the current layout
size_t nvfp4_sf_tiled_bytes(int64_t N, int64_t K);
// exact fp32 export [N][K] of a weight, its scale factors read back from the tiled device layout
void nvfp4_weight_dequant_launch(const Nvfp4Dev& w, float* out, cudaStream_t s);
int32_t nvfp4_gemm_launch(Nvfp4Scratch& scratch, const Nvfp4Dev& w, const uint8_t* a_codes, const uint8_t* a_sf, float ta,
                          int64_t M, uint16_t* c, int device, int sm_count, cudaStream_t s, int* launches, std::string& err);

// launches the tensor-pipe ceiling probe (see nvfp4_mma_probe_kernel); *flop = the flop it executes
int32_t nvfp4_mma_probe_launch(Nvfp4Scratch& scratch, int device, int sm_count, int mmas, cudaStream_t s, double* flop, std::string& err);

}  // namespace mpq
