// NVFP4 block-scaled GEMM for sm_100a: weight build, scale-factor tiling, and a
// persistent warp-specialised TMA + tcgen05 kernel with accumulators in TMEM.
//
//   C[M][N] (bf16) = tsA * tsB * sum_k A~[m,k] * B~[n,k]
//   A~ = e2m1 code * e4m3 scale (one per 16 along K), likewise B~.
//
// No reference source exists for this path (the makepad/makepad snapshot has no
// quantised-linear code); the operator is specified by the task configuration.
//
// TILE.  Output tiles are 224 columns wide (14336 = 64 * 224); a CTA owns 128 rows of one (TMEM has 128 lanes).
// K is consumed in blocks of 256 elements = 128 bytes per row = one 128-byte-swizzle atom = four tcgen05.mma
// (K = 64 each).  Two kernels share that geometry: nvfp4_gemm_pair_kernel_v2 (default; a cluster of two CTAs on
// 256 x 224 tiles with tcgen05 cta_group::2) and nvfp4_gemm_kernel_v2 (one CTA per tile, used where clusters of
// two cannot be scheduled).
//
// ROLES (both kernels).  warp 0: TMA producer.  warp 1: TMEM allocation, MMA issue.  warps 2..9: epilogue
// (tcgen05.ld of the whole accumulator into registers, release, then scale -> bf16 -> global).  warps 10..13:
// scale-factor writers (shared memory -> registers -> TMEM by tcgen05.st).
//
// CODES need no repack: canonical [rows][K/2] bytes are K-major, which is what the MMA's shared-memory descriptor
// (K-major, SWIZZLE_128B) wants; TMA applies the swizzle.  SCALE FACTORS of the weights are re-tiled once into
// 512-byte atoms, one per 128 rows and K step of 64: byte (row%32)*16 + (row/32)*4 + j (j = the step's four scales),
// which is, per TMEM lane, the four columns the tensor core reads; B's slabs are per 224-row tile (two atoms, the
// second three-quarters full).  The activations' scale factors are fetched from their canonical array by TMA
// (16 bytes per row and K block) when K is a multiple of 256, else re-tiled per call like the weights'.
//
// No TMA load here uses cluster multicast.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>

#include "nvfp4.cuh"
#include "swiglu.cuh"
#include "per_device.h"

namespace mpq {

// ---------------------------------------------------------------------------
// exact export
// ---------------------------------------------------------------------------
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

// ---------------------------------------------------------------------------
// activation quantisation: fp32 / bf16 rows -> canonical NVFP4 (what the GEMM takes as A)
// ---------------------------------------------------------------------------
// Per row and 16-element block: amax = max |x|; scale byte = e4m3(amax / (6 * ts)), round to nearest even,
// saturating at 448; each element -> e2m1(x / (e4m3 value * ts)), round to nearest even, saturating at 6; a block
// whose scale encodes to zero gets all-zero codes.  binary32 arithmetic with correctly rounded divisions, so the
// result is the same bit pattern on any IEEE machine.  One thread per block: 64 (32) bytes in, 9 bytes out.
__device__ __forceinline__ uint32_t f32_to_e4m3_sat(float x)          // x >= 0, finite
{
    if (x >= 448.f) return 0x7Eu;
    // grid spacing 2^-9 below 2^-6, else 2^(floor(log2 x) - 3)
    int le = (int)((__float_as_uint(x) >> 23) & 0xFFu) - 127;
    if (le < -6) le = -6;
    const float q = __uint_as_float((uint32_t)(le - 3 + 127) << 23);
    const float y = rintf(__fdiv_rn(x, q)) * q;                        // exact: q is a power of two
    if (y == 0.f) return 0u;
    const int yle = (int)((__float_as_uint(y) >> 23) & 0xFFu) - 127;
    if (yle < -6) return (uint32_t)(y * 512.f);                        // subnormal: mantissa count of 2^-9
    const uint32_t man = (uint32_t)(y * __uint_as_float((uint32_t)(3 - yle + 127) << 23)) - 8u;
    return ((uint32_t)(yle + 7) << 3) | man;
}

__device__ __forceinline__ uint32_t f32_to_e2m1_sat(float f)
{
    const uint32_t sign = (__float_as_uint(f) >> 31) ? 8u : 0u;
    const float x = fabsf(f);
    uint32_t m;
    if (x <= 0.25f) m = 0;
    else if (x < 0.75f) m = 1;
    else if (x <= 1.25f) m = 2;
    else if (x < 1.75f) m = 3;
    else if (x <= 2.5f) m = 4;
    else if (x < 3.5f) m = 5;
    else if (x <= 5.0f) m = 6;
    else m = 7;
    return sign | m;
}

// 16 consecutive elements starting at element `at` of a row-major fp32 or bf16 array
template <bool BF16>
__device__ __forceinline__ void nvfp4_load16(const void* xin, int64_t at, float (&v)[16])
{
    if (BF16) {
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(xin) + at);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const uint4 u = src[q];
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[8 * q + 2 * i] = __uint_as_float(w[i] << 16);
                v[8 * q + 2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
            }
        }
    } else {
        const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(xin) + at);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 f = src[q];
            v[4 * q] = f.x; v[4 * q + 1] = f.y; v[4 * q + 2] = f.z; v[4 * q + 3] = f.w;
        }
    }
}

// SWIGLU: the input is [R][2K] = [gate | up] and what is quantised is silu(gate) * up (fp32), never written to memory.
template <bool BF16, bool SWIGLU>
__global__ void nvfp4_quantize_kernel(const void* __restrict__ xin, int64_t R, int64_t K, float ts, uint8_t* __restrict__ codes,
                                      uint8_t* __restrict__ sf)
{
    const int64_t blk = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (blk >= R * (K / 16)) return;
    float v[16];
    if (SWIGLU) {
        const int64_t r = blk / (K / 16), k0 = (blk - r * (K / 16)) * 16;
        float u[16];
        nvfp4_load16<BF16>(xin, r * 2 * K + k0, v);
        nvfp4_load16<BF16>(xin, r * 2 * K + K + k0, u);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = swiglu_f32(v[i], u[i]);
    } else {
        nvfp4_load16<BF16>(xin, blk * 16, v);
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const uint32_t s8 = f32_to_e4m3_sat(__fdiv_rn(amax, 6.0f * ts));
    const float d = e4m3_value(s8) * ts;
    uint32_t lo = 0, hi = 0;
    if (d > 0.f) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            lo |= f32_to_e2m1_sat(__fdiv_rn(v[i], d)) << (4 * i);
            hi |= f32_to_e2m1_sat(__fdiv_rn(v[8 + i], d)) << (4 * i);
        }
    }
    reinterpret_cast<uint2*>(codes)[blk] = make_uint2(lo, hi);          // element 2j in the low nibble of byte j
    sf[blk] = (uint8_t)s8;
}

void nvfp4_quantize_launch(const void* x, bool bf16, bool swiglu, int64_t R, int64_t K, float ts, uint8_t* codes, uint8_t* sf, cudaStream_t s)
{
    const int64_t blocks = R * (K / 16);
    const unsigned grid = (unsigned)((blocks + 255) / 256);
    if (swiglu) {
        if (bf16) nvfp4_quantize_kernel<true, true><<<grid, 256, 0, s>>>(x, R, K, ts, codes, sf);
        else nvfp4_quantize_kernel<false, true><<<grid, 256, 0, s>>>(x, R, K, ts, codes, sf);
    } else {
        if (bf16) nvfp4_quantize_kernel<true, false><<<grid, 256, 0, s>>>(x, R, K, ts, codes, sf);
        else nvfp4_quantize_kernel<false, false><<<grid, 256, 0, s>>>(x, R, K, ts, codes, sf);
    }
}

// ---------------------------------------------------------------------------
// geometry
// ---------------------------------------------------------------------------
constexpr int BM = 128, BN = 224, BK = 256;               // BK in elements

// The same export for a WEIGHT, whose scale factors exist on the device only in the tiled order the GEMM
// consumes (nvfp4_sf_tile_kernel with tiles of BN rows): reading them back from there proves the tiling pass.
__global__ void nvfp4_dequant_tiled_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ sf_tiled, float ts,
                                           int64_t R, int64_t K, int ksteps_pad, float* __restrict__ out)
{
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = R * (K / 2);
    if (i >= total) return;
    int64_t r = i / (K / 2), kb = i - r * (K / 2);
    uint32_t b = codes[i];
    const int atoms = (BN + 127) / 128;
    int64_t tile = r / BN;
    int local = (int)(r - tile * BN), atom = local >> 7, lrow = local & 127;
    int64_t kstep = kb >> 5;                                  // 64 elements = 32 bytes of codes per K step
    int j = (int)((kb >> 3) & 3);                             // which of the step's four scales
    size_t off = (((size_t)tile * ksteps_pad + kstep) * atoms + atom) * 512 + (lrow & 31) * 16 + (lrow >> 5) * 4 + j;
    float s = e4m3_value(sf_tiled[off]);
    out[r * K + 2 * kb] = e2m1_value(b & 0xF) * s * ts;
    out[r * K + 2 * kb + 1] = e2m1_value(b >> 4) * s * ts;
}
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK / 2;                       // 16384
constexpr int B_BYTES = BN * BK / 2;                       // 28672
constexpr int SFA_BYTES = 4 * 512;                         // four K steps x one 128-row atom
constexpr int SFB_BYTES = 4 * 2 * 512;                     // four K steps x two atoms (224 rows)
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;   // 51200
constexpr int OUT_COLS = 16;                               // columns per TMA store of one epilogue warp (one-CTA kernel)
constexpr int OUT_BYTES = 32 * OUT_COLS * 2;               // 1024: 32 rows of bf16, dense
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 8 * OUT_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int TMEM_COLS = 512;
constexpr uint32_t SPIN_LIMIT = 1u << 22;     // polls of one mbarrier before the kernel gives up and reports it

// scale factors of `rows` rows, tiled for tiles of `tile_rows` rows (128 for A, 224 for B):
// dst[tile][kstep][atom][512] with atom = local_row / 128, zero where row or K step is out of range.
// ksteps_pad = K steps of 64 rounded up to a multiple of 4 (one pipeline stage = four steps).
__global__ void nvfp4_sf_tile_kernel(const uint8_t* __restrict__ sf, int64_t rows, int64_t K, int tile_rows, int atoms,
                                     int ksteps_pad, int64_t total, uint8_t* __restrict__ dst)
{
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;      // one thread per 4 bytes (one row, one K step)
    if (i >= total) return;
    int w = (int)(i & 127);                                          // word inside the 512-byte atom
    int64_t rest = i >> 7;
    int atom = (int)(rest % atoms);
    rest /= atoms;
    int kstep = (int)(rest % ksteps_pad);
    int64_t tile = rest / ksteps_pad;
    int r0 = w >> 2, r1 = w & 3;                                     // byte offset r0*16 + r1*4
    int64_t local = (int64_t)atom * 128 + r1 * 32 + r0;
    int64_t row = tile * tile_rows + local;
    uint32_t v = 0;
    if (local < tile_rows && row < rows && (int64_t)kstep * 64 < K) {
        const uint8_t* src = sf + row * (K / 16) + (int64_t)kstep * 4;
        int64_t nsf = K / 16 - (int64_t)kstep * 4;                   // K is a multiple of 16, maybe not of 64
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (j < nsf) v |= (uint32_t)src[j] << (8 * j);
    }
    reinterpret_cast<uint32_t*>(dst)[i] = v;
}

static inline int ksteps_padded(int64_t K) { return (int)(((K + 63) / 64 + 3) / 4 * 4); }

void nvfp4_weight_dequant_launch(const Nvfp4Dev& w, float* out, cudaStream_t s)
{
    int64_t total = w.N * (w.K / 2);
    nvfp4_dequant_tiled_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(w.codes, w.sf_tiled, w.tensor_scale, w.N, w.K,
                                                                                 ksteps_padded(w.K), out);
}

// tile_multiple: the number of tiles is rounded up to a multiple of it (2 for the activations: a CTA pair always
// loads two 128-row slabs); the extra tiles are zero
static cudaError_t sf_tile_launch(const uint8_t* sf, int64_t rows, int64_t K, int tile_rows, uint8_t* dst, cudaStream_t s, int tile_multiple = 1)
{
    int atoms = (tile_rows + 127) / 128;
    int64_t tiles = (rows + tile_rows - 1) / tile_rows;
    tiles = (tiles + tile_multiple - 1) / tile_multiple * tile_multiple;
    int kp = ksteps_padded(K);
    int64_t total = tiles * kp * atoms * 128;
    nvfp4_sf_tile_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(sf, rows, K, tile_rows, atoms, kp, total, dst);
    return cudaGetLastError();
}

static size_t sf_tiled_bytes(int64_t rows, int64_t K, int tile_rows, int tile_multiple = 1)
{
    int atoms = (tile_rows + 127) / 128;
    int64_t tiles = (rows + tile_rows - 1) / tile_rows;
    tiles = (tiles + tile_multiple - 1) / tile_multiple * tile_multiple;
    return (size_t)tiles * ksteps_padded(K) * atoms * 512;
}

size_t nvfp4_sf_tiled_bytes(int64_t N, int64_t K) { return sf_tiled_bytes(N, K, BN); }

int32_t nvfp4_weight_build(Nvfp4Dev& w, int64_t N, int64_t K, const uint8_t* codes_host, const uint8_t* sf_host, float ts,
                           int* launches, std::string& err)
{
    w.N = N; w.K = K; w.tensor_scale = ts;
    size_t cb = (size_t)N * (K / 2), sb = (size_t)N * (K / 16);
    uint8_t* sf_canonical = nullptr;                      // staging only: the device keeps the tiled copy
    w.sf_tiled_bytes = sf_tiled_bytes(N, K, BN);
    cudaError_t e = cudaMalloc(&w.codes, cb);
    if (e == cudaSuccess) e = cudaMalloc(&sf_canonical, sb);
    if (e == cudaSuccess) e = cudaMalloc(&w.sf_tiled, w.sf_tiled_bytes);
    if (e == cudaSuccess) e = cudaMemcpy(w.codes, codes_host, cb, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(sf_canonical, sf_host, sb, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = sf_tile_launch(sf_canonical, N, K, BN, w.sf_tiled, 0);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaFree(sf_canonical);
    *launches = 1;
    if (e != cudaSuccess) { err = std::string("NVFP4 weight build failed: ") + cudaGetErrorString(e); return MPQ_ERR_CUDA; }
    return MPQ_OK;
}

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t s2u(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// bounded wait: false when the limit ran out
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, uint32_t limit)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .u32 n;\n\t"
        "mov.u32 n, 0;\n\t"
        "W_LOOP:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "@p bra W_DONE;\n\t"
        "add.u32 n, n, 1;\n\t"
        "setp.lt.u32 p, n, %3;\n\t"
        "@p bra W_LOOP;\n\t"
        "mov.u32 %0, 0;\n\t"
        "bra W_END;\n\t"
        "W_DONE:\n\t"
        "mov.u32 %0, 1;\n\t"
        "W_END:\n\t"
        "}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(limit) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                            uint32_t sfb, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t"
        "}"
        ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* r)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
// registers -> this warp's 32 TMEM lanes: thread l writes lane l, register j goes to column +j
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t* r)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
                   "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// TMA tile store shared -> global (rows and columns beyond the tensor are clipped); completion is tracked per thread
// by bulk groups
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, uint32_t src)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x), "r"(y), "r"(src) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ bool bar_test(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded spin on a phase parity without suspending the thread: for the hand-offs whose latency is on the critical path
__device__ __forceinline__ bool bar_spin(uint32_t bar, uint32_t parity, uint32_t limit)
{
    for (uint32_t n = 0; n < limit; ++n) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// K-major operand tile, SWIZZLE_128B: rows are 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);          // start address
    d |= (uint64_t)1 << 16;                         // leading byte offset field (unused for swizzled K-major): 1
    d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset: 8 rows * 128 B
    d |= (uint64_t)1 << 46;                         // descriptor version for sm_100
    d |= (uint64_t)2 << 61;                         // SWIZZLE_128B
    return d;
}

struct GemmParams {
    const uint8_t* sfa;      // tiled
    const uint8_t* sfb;      // tiled
    __nv_bfloat16* C;
    int M, N, K;
    int m_tiles, n_tiles, k_blocks, ksteps_pad;
    float scale;             // tsA * tsB
    int* status;
    int sfa_direct;          // 1: the activations' scale factors are read from their canonical [M][K/16] array (K % 256 == 0)
};

// ---------------------------------------------------------------------------
// one CTA per tile: scale factors written to TMEM by tcgen05.st, one accumulator
// ---------------------------------------------------------------------------
// Measured on B200: the tensor pipe takes what one thread issues strictly in order and queues almost nothing,
// so every tcgen05.cp of scale factors (about 47 cycles each, twelve per K block, when issued from the MMA thread)
// and every cycle the issuing thread spends between two MMAs is a bubble next to 4 x 112 cycles of math.  Here the
// MMA thread issues nothing but MMAs and one commit per K block:
//   * four WRITER warps move the scale factors shared memory -> registers -> TMEM (tcgen05.st, each warp its own
//     lane quarter; every quarter holds the same copy, lane l column c = rows l + 32 c, as tcgen05.cp.32x128b.warpx4
//     would have left it).  One TMEM buffer of 48 columns per pipeline stage: a stage's "full" barrier can only
//     complete after the MMAs of its previous use have been committed, so the buffer is free whenever its stage is.
//   * the MMA thread looks at the NEXT K block's barriers while the third MMA of the current one is running (one
//     non-blocking test: if they are not complete yet, the last MMA and the commit that frees the stage go first).
//   * the 64 columns left beside two accumulators cannot hold four buffers, so there is ONE accumulator of
//     224 columns; eight epilogue warps pull it into registers (112 columns per thread) and release it before
//     they convert and store, which costs a few hundred cycles per tile instead of a second accumulator.
constexpr int V2_THREADS = 448;               // TMA, MMA, 8 epilogue, 4 writer warps
constexpr int V2_SF_COL = BN;                 // 224 .. 415: STAGES buffers of 48 columns
constexpr int V2_SF_COLS = 48;                // [SFB: 4 K steps x 8 | SFA: 4 K steps x 4]
constexpr int V2_EPI_COLS = BN / 2;           // columns per epilogue warp
static_assert(V2_SF_COL + STAGES * V2_SF_COLS <= TMEM_COLS, "scale-factor buffers must fit beside the accumulator");
static_assert(V2_EPI_COLS == 112, "the epilogue loads 3 x 32 + 16 columns");

// One K block's scale factors of this thread's TMEM lane: r[0..31] = B's (K step ks, columns 8 ks .. 8 ks + 7: rows
// lane + 32 c of the 224-row tile), r[32..47] = A's (columns 4 ks + c: rows lane + 32 c).  src points at the stage's
// scale area + 16 * lane.  A's scales are either tiled like B's (512-byte atoms per K step) or, read directly from
// the canonical array by TMA, 128 rows of 16 bytes: row r's four K steps are the four words at 16 r.
__device__ __forceinline__ void load_sf_registers(const unsigned char* src, bool sfa_direct, uint32_t (&r)[48])
{
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
        const uint4 b0 = *reinterpret_cast<const uint4*>(src + SFA_BYTES + ks * 1024);
        const uint4 b1 = *reinterpret_cast<const uint4*>(src + SFA_BYTES + ks * 1024 + 512);
        r[8 * ks + 0] = b0.x; r[8 * ks + 1] = b0.y; r[8 * ks + 2] = b0.z; r[8 * ks + 3] = b0.w;
        r[8 * ks + 4] = b1.x; r[8 * ks + 5] = b1.y; r[8 * ks + 6] = b1.z; r[8 * ks + 7] = b1.w;
    }
    if (sfa_direct) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint4 a = *reinterpret_cast<const uint4*>(src + c * 512);     // row lane + 32 c
            r[32 + c] = a.x; r[36 + c] = a.y; r[40 + c] = a.z; r[44 + c] = a.w;
        }
    } else {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const uint4 a = *reinterpret_cast<const uint4*>(src + ks * 512);
            r[32 + 4 * ks + 0] = a.x; r[32 + 4 * ks + 1] = a.y; r[32 + 4 * ks + 2] = a.z; r[32 + 4 * ks + 3] = a.w;
        }
    }
}

__global__ void __launch_bounds__(V2_THREADS, 1)
nvfp4_gemm_kernel_v2(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_c, const GemmParams p)
{
    extern __shared__ unsigned char smem_dyn[];
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile int s_abort;
    const uint32_t smem0 = (s2u(smem_dyn) + 1023u) & ~1023u;
    const uint32_t out0 = smem0 + STAGES * STAGE_BYTES;              // the epilogue warps' staging tiles
    const uint32_t bars = out0 + 8 * OUT_BYTES;
    const uint32_t bar_full = bars, bar_empty = bars + 8 * STAGES, bar_sf_ready = bars + 16 * STAGES,
                   bar_acc_full = bars + 24 * STAGES, bar_acc_empty = bars + 24 * STAGES + 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = p.m_tiles * p.n_tiles;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) {
            bar_init(bar_full + 8 * s, 1);
            bar_init(bar_empty + 8 * s, 5);        // the MMAs' commit + the four writer warps
            bar_init(bar_sf_ready + 8 * s, 4);
        }
        bar_init(bar_acc_full, 1);
        bar_init(bar_acc_empty, 8);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(&s_tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !s_abort; tile += gridDim.x) {
                const int nt = tile / p.m_tiles, mt = tile - nt * p.m_tiles;
                const uint8_t* sfa_t = p.sfa + (size_t)mt * p.ksteps_pad * 512;
                const uint8_t* sfb_t = p.sfb + (size_t)nt * p.ksteps_pad * 1024;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!bar_wait(bar_empty + 8 * stage, phase ^ 1u, SPIN_LIMIT)) { atomicExch(p.status, 3); s_abort = 1; break; }
                    const uint32_t st = smem0 + stage * STAGE_BYTES, full = bar_full + 8 * stage;
                    bar_expect_tx(full, STAGE_BYTES);
                    tma_load_2d(st, &map_a, kb * (BK / 2), mt * BM, full);
                    tma_load_2d(st + A_BYTES, &map_b, kb * (BK / 2), nt * BN, full);
                    if (p.sfa_direct) tma_load_2d(st + A_BYTES + B_BYTES, &map_sfa, kb * 16, mt * BM, full);   // [128 rows][16 scales]
                    else bulk_load(st + A_BYTES + B_BYTES, sfa_t + (size_t)kb * SFA_BYTES, SFA_BYTES, full);
                    bulk_load(st + A_BYTES + B_BYTES + SFA_BYTES, sfb_t + (size_t)kb * SFB_BYTES, SFB_BYTES, full);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            const int my_tiles = blockIdx.x < total_tiles ? (total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
            const long long total_kb = (long long)my_tiles * p.k_blocks;
            long long done_kb = 0;
            int stage = 0;
            uint32_t phase = 0;
            bool seen = false;                         // the barriers of (stage, phase) have already been observed
            bool ok = true;
            const uint64_t adesc0 = smem_desc_sw128(smem0), bdesc0 = smem_desc_sw128(smem0 + A_BYTES);
            const uint32_t sfc0 = tmem + V2_SF_COL;
            uint32_t soff = 0, sfoff = 0;              // stage * (STAGE_BYTES >> 4), stage * V2_SF_COLS
            for (int local = 0; local < my_tiles && ok && !s_abort; ++local) {
                // the accumulator is free once the eight epilogue warps hold the previous tile in registers
                if (local > 0 && !bar_spin(bar_acc_empty, (uint32_t)(local - 1) & 1u, SPIN_LIMIT)) { atomicExch(p.status, 4); s_abort = 1; break; }
                tc_fence_after();
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!seen) {
                        ok = bar_spin(bar_sf_ready + 8 * stage, phase, SPIN_LIMIT) && bar_spin(bar_full + 8 * stage, phase, SPIN_LIMIT);
                        if (!ok) { atomicExch(p.status, 5); s_abort = 1; break; }
                        tc_fence_after();
                    }
                    seen = false;
                    // Whatever runs between two MMAs must be shorter than one MMA (112 cycles) or the pipe idles: the look at
                    // the next K block's two barriers and the fence are spread over the gaps, the address arithmetic is a few adds.
                    const uint64_t adesc = adesc0 + soff, bdesc = bdesc0 + soff;
                    const uint32_t sfb_c = sfc0 + sfoff, sfa_c = sfb_c + 32;
                    ++done_kb;
                    int nstage = stage + 1;
                    uint32_t nphase = phase;
                    if (nstage == STAGES) { nstage = 0; nphase ^= 1u; }
                    const bool more = done_kb < total_kb;
                    tc_mma_nvf4(tmem, adesc, bdesc, idesc, sfa_c, sfb_c, kb ? 1u : 0u);
                    const bool r1 = more && bar_test(bar_sf_ready + 8 * nstage, nphase);
                    tc_mma_nvf4(tmem, adesc + 2, bdesc + 2, idesc, sfa_c + 4, sfb_c + 8, 1u);        // +32 bytes along K = +2
                    const bool r2 = r1 && bar_test(bar_full + 8 * nstage, nphase);
                    tc_mma_nvf4(tmem, adesc + 4, bdesc + 4, idesc, sfa_c + 8, sfb_c + 16, 1u);
                    if (r2) {
                        tc_fence_after();                  // seen now; if not ready, the last MMA and the commit that frees this
                        seen = true;                       // stage must not wait for it
                    }
                    tc_mma_nvf4(tmem, adesc + 6, bdesc + 6, idesc, sfa_c + 12, sfb_c + 24, 1u);
                    tc_commit(bar_empty + 8 * stage);       // the stage and its scale-factor buffer are free when these MMAs are done
                    soff += STAGE_BYTES >> 4;
                    sfoff += V2_SF_COLS;
                    if (nstage == 0) { soff = 0; sfoff = 0; }
                    stage = nstage;
                    phase = nphase;
                }
                if (!ok) break;
                tc_commit(bar_acc_full);                   // accumulator complete
            }
        }
    } else if (warp >= 10) {
        // ---------------- scale-factor writers: warps 10..13, TMEM lane quarter = warp % 4 ----------------
        const uint32_t lanes = (uint32_t)((warp & 3) * 32) << 16;
        const unsigned char* sf_smem = smem_dyn + (smem0 - s2u(smem_dyn)) + A_BYTES + B_BYTES + lane * 16;
        int stage = 0;
        uint32_t phase = 0;
        bool live = true;
        for (int tile = blockIdx.x; tile < total_tiles && live && !s_abort; tile += gridDim.x) {
            for (int kb = 0; kb < p.k_blocks; ++kb) {
                if (!bar_spin(bar_full + 8 * stage, phase, SPIN_LIMIT)) { if (lane == 0) { atomicExch(p.status, 8); s_abort = 1; } live = false; break; }
                const unsigned char* src = sf_smem + stage * STAGE_BYTES;
                uint32_t r[48];
                load_sf_registers(src, p.sfa_direct != 0, r);
                // full[stage] can only have completed after the MMAs of the stage's previous use were committed:
                // nobody reads this stage's TMEM buffer any more
                tc_fence_after();
                const uint32_t dst = tmem + lanes + V2_SF_COL + stage * V2_SF_COLS;
                tc_st16(dst, r);
                tc_st16(dst + 16, r + 16);
                tc_st16(dst + 32, r + 32);
                tc_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    bar_arrive(bar_sf_ready + 8 * stage);
                    bar_arrive(bar_empty + 8 * stage);         // this warp no longer needs the stage's shared memory
                }
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else {
        // ---------------- epilogue: warps 2..9; TMEM lane quarter = warp % 4, column half = (warp - 2) / 4 ----------------
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        int local = 0;
        for (int tile = blockIdx.x; tile < total_tiles && !s_abort; tile += gridDim.x, ++local) {
            const int nt = tile / p.m_tiles, mt = tile - nt * p.m_tiles;
            if (!bar_spin(bar_acc_full, (uint32_t)local & 1u, SPIN_LIMIT)) { if (lane == 0) { atomicExch(p.status, 6); s_abort = 1; } break; }
            tc_fence_after();
            const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + half * V2_EPI_COLS;
            uint32_t r[V2_EPI_COLS];
            tc_ld32(taddr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
            tc_ld32(taddr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
            tc_ld32(taddr + 64, *reinterpret_cast<uint32_t(*)[32]>(&r[64]));
            tc_ld16(taddr + 96, &r[96]);
            tc_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) bar_arrive(bar_acc_empty);          // the next tile's MMAs may overwrite the accumulator
            // the tile leaves through shared memory as TMA tile stores of 32 rows x 16 columns (see the pair kernel)
            const int row0 = mt * BM + quarter * 32;
            const int col0 = nt * BN + half * V2_EPI_COLS;
            const uint32_t stg = out0 + (uint32_t)(warp - 2) * OUT_BYTES;
#pragma unroll
            for (int round = 0; round < V2_EPI_COLS / OUT_COLS; ++round) {
                if (lane == 0) tma_store_wait_read();              // the previous store has read the staging tile
                __syncwarp();
#pragma unroll
                for (int v = 0; v < OUT_COLS / 8; ++v) {
                    const uint32_t* q = &r[round * OUT_COLS + 8 * v];
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(q[0]) * p.scale, __uint_as_float(q[1]) * p.scale);
                    __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(q[2]) * p.scale, __uint_as_float(q[3]) * p.scale);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(q[4]) * p.scale, __uint_as_float(q[5]) * p.scale);
                    __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(q[6]) * p.scale, __uint_as_float(q[7]) * p.scale);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stg + lane * (OUT_COLS * 2) + v * 16),
                                 "r"(*reinterpret_cast<uint32_t*>(&h0)), "r"(*reinterpret_cast<uint32_t*>(&h1)),
                                 "r"(*reinterpret_cast<uint32_t*>(&h2)), "r"(*reinterpret_cast<uint32_t*>(&h3)) : "memory");
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic writes -> visible to the TMA engine
                __syncwarp();
                if (lane == 0 && row0 < p.M && col0 + round * OUT_COLS < p.N) tma_store_2d(&map_c, col0 + round * OUT_COLS, row0, stg);
            }
        }
        if (lane == 0) tma_store_wait_all();                       // the stores are complete before the CTA exits
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------
// CTA pairs: 256 x 224 tiles, tcgen05 cta_group::2
// ---------------------------------------------------------------------------
// Two CTAs of a cluster share one MMA: the leader (even rank) issues tcgen05.mma.cta_group::2 with M = 256; each CTA
// holds its own 128 rows of A, HALF of the B tile (112 rows) and its own accumulator, so a CTA loads 36 KB per K block
// instead of 51 KB.  The helpers below are the cluster-scope pieces.
constexpr int P_BH_BYTES = (BN / 2) * BK / 2;                                    // 14336: half of the B tile

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// no memory ordering of its own: for hand-offs whose data went through tcgen05 fences (tensor memory), not shared memory
__device__ __forceinline__ void bar_arrive_cluster_relaxed(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void bar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of a CTA pair: the bytes are counted on the barrier of the pair's leader (address with the peer bit cleared)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar & 0xFEFFFFFFu) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4_pair(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                                 uint32_t sfb, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t"
        "}"
        ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate) : "memory");
}

struct PairParams {
    __nv_bfloat16* C;
    int M, N, K;
    int m_pairs, n_tiles, k_blocks, ksteps_pad;   // m_pairs = ceil(M / 256)
    float scale;
    int* status;
    int sfa_direct;          // 1: the activations' scale factors are read from their canonical [M][K/16] array (K % 256 == 0)
};

// ---------------------------------------------------------------------------
// the default kernel where clusters of two can be scheduled
// ---------------------------------------------------------------------------
// nvfp4_gemm_kernel_v2's structure (writer warps, one accumulator drained into registers, look-ahead waits) on
// 256 x 224 tiles of a CTA pair: each CTA loads its 128 rows of A and HALF of the B tile, which cuts the
// L2 -> shared-memory traffic per flop by a third -- with the scale copies out of the way that traffic is what
// bounds the single-CTA kernel.  A and B tiles are TMA loads with .cta_group::2 counted on the LEADER's full
// barrier; the scale-factor slabs are plain bulk copies counted on each CTA's OWN barrier, which is what its
// writer warps wait for; the writers of both CTAs then arrive on the leader's sf_ready barrier.  One TMEM
// scale-factor buffer per pipeline stage: a CTA refills a stage only after the leader's commit for the stage's
// previous use has reached it, so the buffer is free whenever its scale factors arrive.
constexpr int Q_STAGES = 6;
constexpr int Q_STAGE_BYTES = A_BYTES + P_BH_BYTES + SFA_BYTES + SFB_BYTES;     // 36864
constexpr int Q_OUT_COLS = 16;                                                  // columns per TMA store of one epilogue warp
constexpr int Q_OUT_BYTES = 32 * Q_OUT_COLS * 2;                                // 1024: 32 rows of bf16, dense
constexpr int Q_SMEM_BYTES = Q_STAGES * Q_STAGE_BYTES + 8 * Q_OUT_BYTES + 1024 + 256;
static_assert(V2_EPI_COLS % Q_OUT_COLS == 0 && (Q_OUT_COLS * 2) % 16 == 0, "store boxes tile the epilogue columns in 16-byte units");
static_assert(V2_SF_COL + Q_STAGES * V2_SF_COLS <= TMEM_COLS, "scale-factor buffers must fit beside the accumulator");

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(V2_THREADS, 1)
nvfp4_gemm_pair_kernel_v2(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                          const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_c, const PairParams p,
                          const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb)
{
    extern __shared__ unsigned char smem_dyn[];
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile int s_abort;
    const uint32_t smem0 = (s2u(smem_dyn) + 1023u) & ~1023u;
    const uint32_t out0 = smem0 + Q_STAGES * Q_STAGE_BYTES;          // the epilogue warps' staging tiles
    const uint32_t bars = out0 + 8 * Q_OUT_BYTES;
    // full: A and B of both CTAs (leader's is used); sf_full: this CTA's scale slabs; empty: commit + 4 local writers;
    // sf_ready: 8 writer warps of the pair (leader's is used)
    const uint32_t bar_full = bars, bar_sf_full = bars + 8 * Q_STAGES, bar_empty = bars + 16 * Q_STAGES,
                   bar_sf_ready = bars + 24 * Q_STAGES, bar_acc_full = bars + 32 * Q_STAGES, bar_acc_empty = bars + 32 * Q_STAGES + 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                 // 0 = leader of the pair
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int total_tiles = p.m_pairs * p.n_tiles;
    constexpr uint32_t AB_BYTES = A_BYTES + P_BH_BYTES, SF_BYTES = SFA_BYTES + SFB_BYTES;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < Q_STAGES; ++s) {
            bar_init(bar_full + 8 * s, 1);
            bar_init(bar_sf_full + 8 * s, 1);
            bar_init(bar_empty + 8 * s, 5);
            bar_init(bar_sf_ready + 8 * s, 8);
        }
        bar_init(bar_acc_full, 1);
        bar_init(bar_acc_empty, 16);                         // 8 epilogue warps of each CTA
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(&s_tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                      // both CTAs' barriers exist before anyone signals them
    tc_fence_after();
    const uint32_t tmem = s_tmem_base;

    if (warp == 0) {
        // ---------------- producer (both CTAs; the leader arms the shared full barrier) ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int tile = pair; tile < total_tiles && !s_abort; tile += npairs) {
                const int nt = tile / p.m_pairs, mp = tile - nt * p.m_pairs;
                const int mt128 = 2 * mp + (int)rank;
                const uint8_t* sfa_t = sfa + (size_t)mt128 * p.ksteps_pad * 512;
                const uint8_t* sfb_t = sfb + (size_t)nt * p.ksteps_pad * 1024;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!bar_spin(bar_empty + 8 * stage, phase ^ 1u, SPIN_LIMIT)) { atomicExch(p.status, 13); s_abort = 1; break; }
                    const uint32_t st = smem0 + stage * Q_STAGE_BYTES, full = bar_full + 8 * stage, sf_full = bar_sf_full + 8 * stage;
                    bar_expect_tx(sf_full, SF_BYTES);
                    if (p.sfa_direct) tma_load_2d(st + AB_BYTES, &map_sfa, kb * 16, mt128 * BM, sf_full);      // [128 rows][16 scales]
                    else bulk_load(st + AB_BYTES, sfa_t + (size_t)kb * SFA_BYTES, SFA_BYTES, sf_full);
                    bulk_load(st + AB_BYTES + SFA_BYTES, sfb_t + (size_t)kb * SFB_BYTES, SFB_BYTES, sf_full);
                    if (rank == 0) bar_expect_tx(full, 2 * AB_BYTES);
                    tma_load_2d_pair(st, &map_a, kb * (BK / 2), mt128 * BM, full);
                    tma_load_2d_pair(st + A_BYTES, &map_b, kb * (BK / 2), nt * BN + (int)rank * (BN / 2), full);
                    if (++stage == Q_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the leader only ----------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            const int my_tiles = pair < total_tiles ? (total_tiles - 1 - pair) / npairs + 1 : 0;
            const long long total_kb = (long long)my_tiles * p.k_blocks;
            long long done_kb = 0;
            int stage = 0;
            uint32_t phase = 0;
            bool seen = false, ok = true;
            const uint64_t adesc0 = smem_desc_sw128(smem0), bdesc0 = smem_desc_sw128(smem0 + A_BYTES);
            const uint32_t sfc0 = tmem + V2_SF_COL;
            uint32_t soff = 0, sfoff = 0;              // stage * (Q_STAGE_BYTES >> 4), stage * V2_SF_COLS
            for (int local = 0; local < my_tiles && ok && !s_abort; ++local) {
                if (local > 0 && !bar_spin(bar_acc_empty, (uint32_t)(local - 1) & 1u, SPIN_LIMIT)) { atomicExch(p.status, 14); s_abort = 1; break; }
                tc_fence_after();
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!seen) {
                        ok = bar_spin(bar_sf_ready + 8 * stage, phase, SPIN_LIMIT);
                        ok = ok && bar_spin(bar_full + 8 * stage, phase, SPIN_LIMIT);
                        if (!ok) { atomicExch(p.status, 15); s_abort = 1; break; }
                        tc_fence_after();
                    }
                    seen = false;
                    // Whatever runs between two MMAs must be shorter than one MMA (112 cycles) or the pipe idles: the look at
                    // the next K block's two barriers and the fence are spread over the gaps, the address arithmetic is a few adds.
                    const uint64_t adesc = adesc0 + soff, bdesc = bdesc0 + soff;
                    const uint32_t sfb_c = sfc0 + sfoff, sfa_c = sfb_c + 32;
                    ++done_kb;
                    int nstage = stage + 1;
                    uint32_t nphase = phase;
                    if (nstage == Q_STAGES) { nstage = 0; nphase ^= 1u; }
                    const bool more = done_kb < total_kb;
                    tc_mma_nvf4_pair(tmem, adesc, bdesc, idesc, sfa_c, sfb_c, kb ? 1u : 0u);
                    const bool r1 = more && bar_test(bar_sf_ready + 8 * nstage, nphase);
                    tc_mma_nvf4_pair(tmem, adesc + 2, bdesc + 2, idesc, sfa_c + 4, sfb_c + 8, 1u);        // +32 bytes along K = +2
                    const bool r2 = r1 && bar_test(bar_full + 8 * nstage, nphase);
                    tc_mma_nvf4_pair(tmem, adesc + 4, bdesc + 4, idesc, sfa_c + 8, sfb_c + 16, 1u);
                    if (r2) {
                        tc_fence_after();                  // seen now; if not ready, the last MMA and the commit that frees this
                        seen = true;                       // stage must not wait for it
                    }
                    tc_mma_nvf4_pair(tmem, adesc + 6, bdesc + 6, idesc, sfa_c + 12, sfb_c + 24, 1u);
                    tc_commit_pair(bar_empty + 8 * stage);       // the stage and its scale-factor buffer are free when these MMAs are done
                    soff += Q_STAGE_BYTES >> 4;
                    sfoff += V2_SF_COLS;
                    if (nstage == 0) { soff = 0; sfoff = 0; }
                    stage = nstage;
                    phase = nphase;
                }
                if (!ok) break;
                tc_commit_pair(bar_acc_full);                    // both CTAs' epilogues may read
            }
        }
    } else if (warp >= 10) {
        // ---------------- scale-factor writers: warps 10..13 of each CTA, TMEM lane quarter = warp % 4 ----------------
        const uint32_t lanes = (uint32_t)((warp & 3) * 32) << 16;
        const unsigned char* sf_smem = smem_dyn + (smem0 - s2u(smem_dyn)) + AB_BYTES + lane * 16;
        const uint32_t leader_sf_ready = map_to_cta(bar_sf_ready, 0);
        int stage = 0;
        uint32_t phase = 0;
        bool live = true;
        for (int tile = pair; tile < total_tiles && live && !s_abort; tile += npairs) {
            for (int kb = 0; kb < p.k_blocks; ++kb) {
                if (!bar_spin(bar_sf_full + 8 * stage, phase, SPIN_LIMIT)) { if (lane == 0) { atomicExch(p.status, 18); s_abort = 1; } live = false; break; }
                const unsigned char* src = sf_smem + stage * Q_STAGE_BYTES;
                uint32_t r[48];
                load_sf_registers(src, p.sfa_direct != 0, r);
                tc_fence_after();
                const uint32_t dst = tmem + lanes + V2_SF_COL + stage * V2_SF_COLS;
                tc_st16(dst, r);
                tc_st16(dst + 16, r + 16);
                tc_st16(dst + 32, r + 32);
                tc_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (rank == 0) bar_arrive(bar_sf_ready + 8 * stage);
                    else bar_arrive_cluster_relaxed(leader_sf_ready + 8 * stage);
                    bar_arrive(bar_empty + 8 * stage);
                }
                if (++stage == Q_STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else {
        // ---------------- epilogue: warps 2..9 of each CTA, its own 128 rows ----------------
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const uint32_t leader_acc_empty = map_to_cta(bar_acc_empty, 0);
        int local = 0;
        for (int tile = pair; tile < total_tiles && !s_abort; tile += npairs, ++local) {
            const int nt = tile / p.m_pairs, mp = tile - nt * p.m_pairs;
            if (!bar_spin(bar_acc_full, (uint32_t)local & 1u, SPIN_LIMIT)) { if (lane == 0) { atomicExch(p.status, 16); s_abort = 1; } break; }
            tc_fence_after();
            const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + half * V2_EPI_COLS;
            uint32_t r[V2_EPI_COLS];
            tc_ld32(taddr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
            tc_ld32(taddr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
            tc_ld32(taddr + 64, *reinterpret_cast<uint32_t(*)[32]>(&r[64]));
            tc_ld16(taddr + 96, &r[96]);
            tc_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {                                       // the leader's MMA thread waits for all sixteen warps
                if (rank == 0) bar_arrive(bar_acc_empty);
                else bar_arrive_cluster_relaxed(leader_acc_empty);
            }
            // Stores: one lane per row would touch 32 rows with every instruction, and all CTAs store at the same time
            // (the tile boundaries coincide): measured, that stalls the next tile's loads for 2-3 us.  So the tile goes
            // through shared memory and leaves as TMA tile stores of 32 rows x Q_OUT_COLS columns.
            const int row0 = (2 * mp + (int)rank) * BM + quarter * 32;
            const int col0 = nt * BN + half * V2_EPI_COLS;
            const uint32_t stg = out0 + (uint32_t)(warp - 2) * Q_OUT_BYTES;
#pragma unroll
            for (int round = 0; round < V2_EPI_COLS / Q_OUT_COLS; ++round) {
                if (lane == 0) tma_store_wait_read();              // the previous store has read the staging tile
                __syncwarp();
#pragma unroll
                for (int v = 0; v < Q_OUT_COLS / 8; ++v) {
                    const uint32_t* q = &r[round * Q_OUT_COLS + 8 * v];
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(q[0]) * p.scale, __uint_as_float(q[1]) * p.scale);
                    __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(q[2]) * p.scale, __uint_as_float(q[3]) * p.scale);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(q[4]) * p.scale, __uint_as_float(q[5]) * p.scale);
                    __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(q[6]) * p.scale, __uint_as_float(q[7]) * p.scale);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stg + lane * (Q_OUT_COLS * 2) + v * 16),
                                 "r"(*reinterpret_cast<uint32_t*>(&h0)), "r"(*reinterpret_cast<uint32_t*>(&h1)),
                                 "r"(*reinterpret_cast<uint32_t*>(&h2)), "r"(*reinterpret_cast<uint32_t*>(&h3)) : "memory");
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic writes -> visible to the TMA engine
                __syncwarp();
                if (lane == 0 && row0 < p.M && col0 + round * Q_OUT_COLS < p.N) tma_store_2d(&map_c, col0 + round * Q_OUT_COLS, row0, stg);
            }
        }
        if (lane == 0) tma_store_wait_all();                       // the stores are complete before the CTA exits
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                      // the peer's shared memory and barriers stay valid until both are done
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------
// measured ceiling of the FP4 tensor pipe
// ---------------------------------------------------------------------------
// One CTA per SM issues `mmas` block-scaled FP4 MMAs of the GEMM's own shape (128 x 224 x 64, operands in shared
// memory, scale factors in TMEM) back to back, with no loads, no hand-offs and one commit at the end: what the
// tensor pipe sustains when nothing else is in its way.  2 * 128 * 224 * 64 flop per MMA and CTA.
__global__ void __launch_bounds__(128, 1) nvfp4_mma_probe_kernel(int mmas, int* status)
{
    extern __shared__ unsigned char smem_dyn[];
    __shared__ uint32_t s_tmem_base;
    const uint32_t smem0 = (s2u(smem_dyn) + 1023u) & ~1023u;
    const uint32_t bar = smem0 + A_BYTES + B_BYTES;
    const int warp = threadIdx.x >> 5;
    // operands: every byte 0x22 (two e2m1 codes of value 1.0); any bit pattern is a valid operand
    for (uint32_t i = threadIdx.x * 16; i < (uint32_t)(A_BYTES + B_BYTES); i += blockDim.x * 16)
        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(smem0 + i), "r"(0x22222222u) : "memory");
    if (threadIdx.x == 0) {
        bar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(&s_tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem_base;
    {   // scale factors 1.0 (e4m3 0x38) in 48 columns beside the accumulator, every lane quarter its own copy
        uint32_t r[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) r[i] = 0x38383838u;
        const uint32_t dst = tmem + ((uint32_t)(warp * 32) << 16) + V2_SF_COL;
        tc_st16(dst, r); tc_st16(dst + 16, r); tc_st16(dst + 32, r);
        tc_st_wait();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (threadIdx.x == 0) {
        const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
        const uint64_t adesc = smem_desc_sw128(smem0), bdesc = smem_desc_sw128(smem0 + A_BYTES);
        const uint32_t sfb_c = tmem + V2_SF_COL, sfa_c = sfb_c + 32;
        for (int i = 0; i < mmas; i += 4) {
            tc_mma_nvf4(tmem, adesc, bdesc, idesc, sfa_c, sfb_c, i ? 1u : 0u);
            tc_mma_nvf4(tmem, adesc + 2, bdesc + 2, idesc, sfa_c + 4, sfb_c + 8, 1u);
            tc_mma_nvf4(tmem, adesc + 4, bdesc + 4, idesc, sfa_c + 8, sfb_c + 16, 1u);
            tc_mma_nvf4(tmem, adesc + 6, bdesc + 6, idesc, sfa_c + 12, sfb_c + 24, 1u);
        }
        tc_commit(bar);
        if (!bar_wait(bar, 0u, SPIN_LIMIT)) atomicExch(status, 21);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

int32_t nvfp4_mma_probe_launch(Nvfp4Scratch& scratch, int device, int sm_count, int mmas, cudaStream_t s, double* flop, std::string& err)
{
    if (!scratch.status) {
        cudaError_t e = cudaMalloc(&scratch.status, sizeof(int));
        if (e == cudaSuccess) e = cudaMemset(scratch.status, 0, sizeof(int));
        if (e != cudaSuccess) { err = std::string("status allocation failed: ") + cudaGetErrorString(e); return MPQ_ERR_CUDA; }
    }
    const int smem = A_BYTES + B_BYTES + 1024 + 64;
    static PerDeviceOnce configured;
    if (configured.needs(device)) {
        cudaError_t e = cudaFuncSetAttribute(nvfp4_mma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) { err = std::string("cudaFuncSetAttribute failed: ") + cudaGetErrorString(e); return MPQ_ERR_CUDA; }
        configured.mark(device);
    }
    mmas = (mmas + 3) / 4 * 4;
    nvfp4_mma_probe_kernel<<<sm_count, 128, smem, s>>>(mmas, scratch.status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { err = std::string("nvfp4_mma_probe_kernel launch failed: ") + cudaGetErrorString(e); return MPQ_ERR_CUDA; }
    if (flop) *flop = 2.0 * BM * BN * 64 * (double)mmas * sm_count;
    return MPQ_OK;
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// rows x (K/2) bytes, K contiguous; box = box_rows x 128 bytes; 128-byte swizzle; out-of-range reads return zero
static bool make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int box_rows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)(K / 2), (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(K / 2)};
    cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// canonical scale factors [rows][K/16] bytes; box = 128 rows x 16 bytes (one K block), no swizzle, zero fill
static bool make_sf_direct_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)(K / 16), (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(K / 16)};
    cuuint32_t box[2] = {16u, (cuuint32_t)BM};
    cuuint32_t estr[2] = {1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}


// C[M][N] bf16; box = 32 rows x box_cols columns, dense
static bool make_c_map(CUtensorMap* map, void* base, int64_t M, int64_t N, int box_cols)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    cuuint64_t strides[1] = {(cuuint64_t)N * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, 32u};
    cuuint32_t estr[2] = {1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// CTA pairs the device can keep resident at once (0: the pair kernel cannot be used)

static int pair_v2_clusters(int device, int sm_count)
{
    static int cached_n[PerDeviceOnce::MAX_DEVICES];      // per device: the attribute and the occupancy both are
    static PerDeviceOnce known;
    if (!known.needs(device)) return cached_n[device];
    int& cached = (device >= 0 && device < PerDeviceOnce::MAX_DEVICES) ? cached_n[device] : cached_n[0];
    known.mark(device);
    cached = 0;
    if (cudaFuncSetAttribute(nvfp4_gemm_pair_kernel_v2, cudaFuncAttributeMaxDynamicSharedMemorySize, Q_SMEM_BYTES) != cudaSuccess) { cudaGetLastError(); return 0; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(sm_count & ~1));
    cfg.blockDim = dim3(V2_THREADS);
    cfg.dynamicSmemBytes = Q_SMEM_BYTES;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, nvfp4_gemm_pair_kernel_v2, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
    cached = n;
    return cached;
}

int32_t nvfp4_gemm_launch(Nvfp4Scratch& scratch, const Nvfp4Dev& w, const uint8_t* a_codes, const uint8_t* a_sf, float ta,
                          int64_t M, uint16_t* c, int device, int sm_count, cudaStream_t s, int* launches, std::string& err)
{
    *launches = 0;
    const int64_t N = w.N, K = w.K;
    if (!scratch.status) {
        cudaError_t e = cudaMalloc(&scratch.status, sizeof(int));
        if (e == cudaSuccess) e = cudaMemset(scratch.status, 0, sizeof(int));
        if (e != cudaSuccess) { err = std::string("status allocation failed: ") + cudaGetErrorString(e); return MPQ_ERR_CUDA; }
    }
    // The activations' scale factors are read straight from the canonical [M][K/16] array when a K block's 16 bytes per
    // row can be a TMA box (row pitch a multiple of 16 bytes); otherwise they are re-tiled first, like the weights'.
    const bool direct = K % 256 == 0 && (reinterpret_cast<uintptr_t>(a_sf) & 15u) == 0;
    cudaError_t e = cudaSuccess;
    if (!direct) {
        size_t need = sf_tiled_bytes(M, K, BM, 2);
        if (scratch.sfa_bytes < need) {
            cudaDeviceSynchronize();
            cudaFree(scratch.sfa_tiled);
            scratch.sfa_tiled = nullptr;
            scratch.sfa_bytes = 0;
            e = cudaMalloc(&scratch.sfa_tiled, need);
            if (e != cudaSuccess) { err = std::string("scratch allocation failed: ") + cudaGetErrorString(e); return MPQ_ERR_CUDA; }
            scratch.sfa_bytes = need;
        }
        e = sf_tile_launch(a_sf, M, K, BM, scratch.sfa_tiled, s, 2);
        *launches += 1;
        if (e != cudaSuccess) { err = std::string("scale-factor tiling failed: ") + cudaGetErrorString(e); return MPQ_ERR_CUDA; }
    }

    CUtensorMap map_a, map_sfa;
    if (!make_map(&map_a, a_codes, M, K, BM) || !(direct ? make_sf_direct_map(&map_sfa, a_sf, M, K) : make_map(&map_sfa, a_codes, M, K, BM))) {
        err = "cuTensorMapEncodeTiled failed (pointers must be 16-byte aligned, K a multiple of 32)";
        return MPQ_ERR_CUDA;
    }
    // CTA pairs where clusters of two can be scheduled (MPQ_FP4_KERNEL=single forces the one-CTA kernel, which the
    // parity tests use to cover both)
    const char* env = getenv("MPQ_FP4_KERNEL");
    const int nclusters = (env && std::string(env) == "single") ? 0 : pair_v2_clusters(device, sm_count);
    if (nclusters > 0) {
        CUtensorMap map_bh, map_c;
        if (!make_map(&map_bh, w.codes, N, K, BN / 2) || !make_c_map(&map_c, c, M, N, Q_OUT_COLS)) { err = "cuTensorMapEncodeTiled failed for the CTA-pair kernel"; return MPQ_ERR_CUDA; }
        PairParams pp;
        pp.C = reinterpret_cast<__nv_bfloat16*>(c);
        pp.M = (int)M; pp.N = (int)N; pp.K = (int)K;
        pp.m_pairs = (int)((M + 2 * BM - 1) / (2 * BM)); pp.n_tiles = (int)((N + BN - 1) / BN);
        pp.k_blocks = (int)((K + BK - 1) / BK); pp.ksteps_pad = ksteps_padded(K);
        pp.scale = ta * w.tensor_scale;
        pp.status = scratch.status;
        pp.sfa_direct = direct ? 1 : 0;
        int grid = 2 * std::min(nclusters, pp.m_pairs * pp.n_tiles);
        nvfp4_gemm_pair_kernel_v2<<<grid, V2_THREADS, Q_SMEM_BYTES, s>>>(map_a, map_bh, map_sfa, map_c, pp, scratch.sfa_tiled, w.sf_tiled);
        *launches += 1;
        e = cudaGetLastError();
        if (e != cudaSuccess) { err = std::string("nvfp4_gemm_pair_kernel_v2 launch failed: ") + cudaGetErrorString(e); return MPQ_ERR_CUDA; }
        return MPQ_OK;
    }
    CUtensorMap map_b, map_c1;
    if (!make_map(&map_b, w.codes, N, K, BN) || !make_c_map(&map_c1, c, M, N, OUT_COLS)) { err = "cuTensorMapEncodeTiled failed"; return MPQ_ERR_CUDA; }
    GemmParams p;
    p.sfa = scratch.sfa_tiled; p.sfb = w.sf_tiled; p.C = reinterpret_cast<__nv_bfloat16*>(c);
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.m_tiles = (int)((M + BM - 1) / BM); p.n_tiles = (int)((N + BN - 1) / BN);
    p.k_blocks = (int)((K + BK - 1) / BK); p.ksteps_pad = ksteps_padded(K);
    p.scale = ta * w.tensor_scale;
    p.status = scratch.status;
    p.sfa_direct = direct ? 1 : 0;
    static PerDeviceOnce configured;
    if (configured.needs(device)) {
        e = cudaFuncSetAttribute(nvfp4_gemm_kernel_v2, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) { err = std::string("cudaFuncSetAttribute failed: ") + cudaGetErrorString(e); return MPQ_ERR_CUDA; }
        configured.mark(device);
    }
    int grid = std::min(sm_count, p.m_tiles * p.n_tiles);
    nvfp4_gemm_kernel_v2<<<grid, V2_THREADS, SMEM_BYTES, s>>>(map_a, map_b, map_sfa, map_c1, p);
    *launches += 1;
    e = cudaGetLastError();
    if (e != cudaSuccess) { err = std::string("nvfp4_gemm_kernel_v2 launch failed: ") + cudaGetErrorString(e); return MPQ_ERR_CUDA; }
    return MPQ_OK;
}

}  // namespace mpq
