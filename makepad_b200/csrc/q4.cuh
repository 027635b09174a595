// Q4 (32-wide blocks, fp16 scale) weights on the device: layout, repack,
// exact export, and the HBM-bound linear kernel for M <= 16 activation rows.
//
// No reference source exists for this path (the makepad/makepad snapshot has no
// quantised-linear code); the operator is specified by the task configuration:
// 4-bit signed codes in [-8,7], two per byte along K, fp16 scale per 32.
//
// DEVICE LAYOUT ("tile stream").  Rows are padded to a multiple of 32 and K to
// a multiple of 64.  A *unit* is one row pair-tile (32 rows = two m16 tiles) by
// one 64-wide K chunk, stored as 1152 contiguous bytes: tile0 codes (512 B),
// tile1 codes (512 B), scales (128 B):
//   codes  inside a tile lane l = 4g+t owns the 16 bytes at l*16 = words q0..q3, one word per
//          m16n8k16 MMA of the chunk.  Nibble i of word qj holds the OFFSET code
//          n = code+8 of
//              row  = tile*16 + g + 8*(i&1)
//              kk   = 16*j + 2t + (i>>2) + 8*((i>>1)&1)        (k inside the chunk)
//          so that (w & 0x000F000F), (w & 0x00F000F0), ((w>>8) & 0x000F000F),
//          ((w>>8) & 0x00F000F0) are, as half2 bit patterns, exactly the four
//          A-fragment registers of mma.m16n8k16 (rows g / g+8, k 2t..2t+1 / +8).
//   scales lane group g owns 16 B = 8 halves
//          [tile][row g | row g+8][block 0 | block 1].
// Units are ordered (row pair, chunk): the whole matrix is ONE contiguous
// stream, and any run of units is a contiguous byte range that a bulk copy
// (cp.async.bulk) can bring into shared memory.
//
// ARITHMETIC.  The masked words are fp16 SUBNORMALS n*2^-24 (rows g) and
// 16n*2^-24 (rows g+8): no conversion instruction is spent on the weights.
// x is split as hi+lo fp16 (22 significant bits) after a per-CTA power-of-two
// renormalisation, hi and lo sit in adjacent B columns, and the -8 offset is
// folded into the MMA's C operand as -8*2^-24*sum_block(x).  One MMA pair per
// 32-block accumulates in fp32; the block's fp16 scale multiplies the pair's
// result in fp32.  Padded rows / K carry code 0 and scale 0.
#pragma once
#include "swiglu.cuh"
#include <cooperative_groups.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mpq {
namespace cg = cooperative_groups;

struct Q4Dev {
    int64_t N = 0, K = 0;      // logical shape of this (shard of the) matrix
    int nrp = 0;               // row pair-tiles  = ceil(N/32)
    int nchunks = 0;           // 64-wide K chunks = ceil(K/64)
    uint4* stream = nullptr;   // nrp*nchunks units of Q4_UNIT_BYTES
    int64_t units() const { return (int64_t)nrp * nchunks; }
    size_t bytes() const { return (size_t)nrp * nchunks * 1152; }
};

constexpr int Q4_UNIT_BYTES = 1152;
constexpr int Q4_UNIT_U4 = Q4_UNIT_BYTES / 16;   // 72 uint4 per unit: 32 + 32 codes, 8 scales

constexpr int Q4_WARPS = 8;     // warps per CTA of the phase-staged kernel (q4_linear_kernel)
constexpr int Q4_THREADS = Q4_WARPS * 32;
constexpr int Q4_PF = 4;       // chunk loads in flight per warp of that kernel

// ---------------------------------------------------------------------------
// repack: canonical -> tile stream.  One thread per 32-bit code word.
// (row0, k0) is the origin of the shard inside the canonical matrix whose row
// pitch is Kfull: a column shard starts at row0, a row shard at k0.
// ---------------------------------------------------------------------------
__global__ void q4_repack_codes_kernel(const uint8_t* __restrict__ codes, int64_t Kfull, int64_t row0, int64_t k0,
                                       int64_t N, int64_t K, int nrp, int nchunks, uint32_t* __restrict__ out)
{
    int64_t W = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = (int64_t)nrp * nchunks * 256;
    if (W >= total) return;
    int j = (int)(W & 3), lane = (int)((W >> 2) & 31), tile = (int)((W >> 7) & 1);
    int64_t unit = W >> 8;
    int ch = (int)(unit % nchunks);
    int64_t rp = unit / nchunks;
    int g = lane >> 2, t = lane & 3;
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int64_t row = rp * 32 + tile * 16 + g + 8 * (i & 1);
        int64_t k = (int64_t)ch * 64 + 16 * j + 2 * t + (i >> 2) + 8 * ((i >> 1) & 1);
        uint32_t n = 8;                                   // code 0
        if (row < N && k < K) {
            uint8_t b = codes[(row0 + row) * (Kfull / 2) + ((k0 + k) >> 1)];
            uint32_t nib = ((k0 + k) & 1) ? (b >> 4) : (b & 0xF);
            n = nib ^ 8;                                  // two's complement -> offset binary
        }
        word |= n << (4 * i);
    }
    out[unit * (Q4_UNIT_BYTES / 4) + (W & 255)] = word;
}

__global__ void q4_repack_scales_kernel(const uint16_t* __restrict__ scales, int64_t KBfull, int64_t row0, int64_t kb0,
                                        int64_t N, int64_t KB, int nrp, int nchunks, uint16_t* __restrict__ out)
{
    int64_t H = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = (int64_t)nrp * nchunks * 64;
    if (H >= total) return;
    int blk = (int)(H & 1), rowsel = (int)((H >> 1) & 1), tile = (int)((H >> 2) & 1), g = (int)((H >> 3) & 7);
    int64_t unit = H >> 6;
    int ch = (int)(unit % nchunks);
    int64_t rp = unit / nchunks;
    int64_t row = rp * 32 + tile * 16 + g + 8 * rowsel;
    int64_t b = (int64_t)ch * 2 + blk;
    out[unit * (Q4_UNIT_BYTES / 2) + 512 + (H & 63)] = (row < N && b < KB) ? scales[(row0 + row) * KBfull + kb0 + b] : (uint16_t)0;
}

// exact fp32 export from the tile stream: out[row][k] = fp32(scale) * fp32(code)
__global__ void q4_dequant_kernel(const uint32_t* __restrict__ stream, int64_t N, int64_t K, int nrp, int nchunks,
                                  float* __restrict__ out)
{
    int64_t W = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = (int64_t)nrp * nchunks * 256;
    if (W >= total) return;
    int j = (int)(W & 3), lane = (int)((W >> 2) & 31), tile = (int)((W >> 7) & 1);
    int64_t unit = W >> 8;
    int ch = (int)(unit % nchunks);
    int64_t rp = unit / nchunks;
    int g = lane >> 2, t = lane & 3;
    uint32_t word = stream[unit * (Q4_UNIT_BYTES / 4) + (W & 255)];
    const uint16_t* scales = reinterpret_cast<const uint16_t*>(stream + unit * (Q4_UNIT_BYTES / 4)) + 512;
    int blk = j >> 1;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int rowsel = i & 1;
        int64_t row = rp * 32 + tile * 16 + g + 8 * rowsel;
        int64_t k = (int64_t)ch * 64 + 16 * j + 2 * t + (i >> 2) + 8 * ((i >> 1) & 1);
        if (row < N && k < K) {
            uint16_t sb = scales[g * 8 + tile * 4 + rowsel * 2 + blk];
            float s = __half2float(__ushort_as_half(sb));
            int code = (int)((word >> (4 * i)) & 0xF) - 8;
            out[row * K + k] = s * (float)code;
        }
    }
}

// ---------------------------------------------------------------------------
// the linear kernel
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_stream(const uint4* p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                         float c0, float c1, float c2, float c3)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c0), "f"(c1), "f"(c2), "f"(c3));
}

// A-fragment of one code word.  SUBN: subnormal halves n*2^-24 / 16n*2^-24.
// Otherwise exact signed halves (code) via the 1024+n magic number.
template <bool SUBN>
__device__ __forceinline__ void q4_unpack(uint32_t w, uint32_t (&a)[4])
{
    uint32_t w8 = w >> 8;
    if (SUBN) {
        a[0] = w & 0x000F000Fu;
        a[1] = w & 0x00F000F0u;
        a[2] = w8 & 0x000F000Fu;
        a[3] = w8 & 0x00F000F0u;
    } else {
        const __half2 k1032 = __floats2half2_rn(1032.f, 1032.f);
        const __half2 k16th = __floats2half2_rn(0.0625f, 0.0625f);
        const __half2 km72 = __floats2half2_rn(-72.f, -72.f);
        uint32_t u0 = (w & 0x000F000Fu) | 0x64006400u, u1 = (w & 0x00F000F0u) | 0x64006400u;
        uint32_t u2 = (w8 & 0x000F000Fu) | 0x64006400u, u3 = (w8 & 0x00F000F0u) | 0x64006400u;
        __half2 h0 = __hsub2(*reinterpret_cast<__half2*>(&u0), k1032);
        __half2 h1 = __hfma2(*reinterpret_cast<__half2*>(&u1), k16th, km72);
        __half2 h2 = __hsub2(*reinterpret_cast<__half2*>(&u2), k1032);
        __half2 h3 = __hfma2(*reinterpret_cast<__half2*>(&u3), k16th, km72);
        a[0] = *reinterpret_cast<uint32_t*>(&h0);
        a[1] = *reinterpret_cast<uint32_t*>(&h1);
        a[2] = *reinterpret_cast<uint32_t*>(&h2);
        a[3] = *reinterpret_cast<uint32_t*>(&h3);
    }
}

struct Q4Launch {
    const uint4* stream;
    const float* X;        // [M][K]
    float* Y;              // [M][ldy]
    int M, N, K;
    int64_t ldy;           // row pitch of Y in floats
    int nchunks;           // chunks per row pair-tile in the stream
    int chunks_per_cta;    // K split: CTA (x, y) covers chunks [y*cpc, (y+1)*cpc)
    int chunks_per_phase;  // chunks of x staged in shared memory at once
    int splits;            // gridDim.y == cluster size along y
};

// dynamic shared memory: xs (B fragments) then cs (C corrections)
//   xs: uint4 [blocks_in_phase][2M columns][4 t]     column 2m = hi, 2m+1 = lo of row m
//   cs: float4[blocks_in_phase][MT][4 t]             (c_hi, c_lo, 16 c_hi, 16 c_lo) for m = 4*bt + t
template <int MT, bool SUBN>
__global__ void __launch_bounds__(Q4_THREADS) q4_linear_kernel(const Q4Launch p)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ float red[Q4_WARPS][4 * MT][32];
    __shared__ float part[4 * MT][32];
    __shared__ uint32_t s_max[Q4_WARPS];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int M = p.M, ncols = 2 * M;
    const int cbeg = min(p.nchunks, (int)blockIdx.y * p.chunks_per_cta);
    const int cend = min(p.nchunks, cbeg + p.chunks_per_cta);
    const int cpp = p.chunks_per_phase;
    uint4* xs = reinterpret_cast<uint4*>(smem_raw);
    float4* cs = reinterpret_cast<float4*>(smem_raw + (size_t)cpp * 2 * ncols * 64);

    const uint4* wbase = p.stream + ((size_t)blockIdx.x * p.nchunks) * Q4_UNIT_U4 + lane;   // + chunk*72 (+32 for tile 1)
    const uint4* sbase = wbase - lane + 64 + g;                                             // + chunk*72

    float acc[2][MT][2];      // [tile][btile][row g | row g+8], summed over phases (already un-normalised)
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < MT; ++b) acc[a][b][0] = acc[a][b][1] = 0.f;

    if (SUBN) {   // corrections of padded activation rows (m >= M) stay zero for the whole kernel
        for (int i = tid; i < cpp * 2 * MT * 4; i += Q4_THREADS) cs[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }

    // let the next kernel in the stream start its own weight prefetch early
    asm volatile("griddepcontrol.launch_dependents;");

    bool waited = false;
    for (int ph0 = cbeg; ph0 < cend; ph0 += cpp) {
        const int ph1 = min(cend, ph0 + cpp);
        // ---- prefetch this warp's first chunks of the phase (weights do not depend on x)
        uint4 wq[Q4_PF][2], sq[Q4_PF];
#pragma unroll
        for (int s = 0; s < Q4_PF; ++s) {
            int c = ph0 + warp + s * Q4_WARPS;
            if (c < ph1) {
                wq[s][0] = ldg_stream(wbase + (size_t)c * Q4_UNIT_U4);
                wq[s][1] = ldg_stream(wbase + (size_t)c * Q4_UNIT_U4 + 32);
                sq[s] = ldg_stream(sbase + (size_t)c * Q4_UNIT_U4);
            }
        }
        if (!waited) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
        __syncthreads();                                   // previous phase fully consumed

        // ---- stage x[:, ph0*64 .. ph1*64) as normalised hi/lo fp16 B fragments
        const int pk4 = (ph1 - ph0) * 16;                  // float4 per activation row in this phase
        const int total4 = M * pk4;
        const int64_t kbase = (int64_t)ph0 * 64;
        uint32_t mx = 0;
        for (int i = tid; i < total4; i += Q4_THREADS) {
            int m = i / pk4, f = i - m * pk4;
            int64_t k = kbase + 4 * f;
            if (k < p.K) {
                float4 v = *reinterpret_cast<const float4*>(p.X + (size_t)m * p.K + k);
                mx = max(mx, __float_as_uint(v.x) & 0x7FFFFFFFu);
                mx = max(mx, __float_as_uint(v.y) & 0x7FFFFFFFu);
                mx = max(mx, __float_as_uint(v.z) & 0x7FFFFFFFu);
                mx = max(mx, __float_as_uint(v.w) & 0x7FFFFFFFu);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        if (lane == 0) s_max[warp] = mx;
        __syncthreads();
        mx = s_max[0];
#pragma unroll
        for (int w = 1; w < Q4_WARPS; ++w) mx = max(mx, s_max[w]);
        // scale = 2^(14 - floor(log2 max)) puts the largest |x| in [2^14, 2^15)
        int emax = (int)(mx >> 23);
        float sc = 1.f, inv_sc = 1.f;
        if (mx != 0 && emax < 255) {
            emax = max(emax, 16);
            sc = __uint_as_float((uint32_t)(268 - emax) << 23);
            inv_sc = __uint_as_float((uint32_t)(emax - 14) << 23);
        }
        const int iters = (total4 + Q4_THREADS - 1) / Q4_THREADS;
        for (int it = 0; it < iters; ++it) {
            int i = it * Q4_THREADS + tid;
            bool on = i < total4;
            int m = on ? i / pk4 : 0, f = on ? i - m * pk4 : 0;
            int64_t k = kbase + 4 * f;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (on && k < p.K) v = *reinterpret_cast<const float4*>(p.X + (size_t)m * p.K + k);
            float e[4] = {v.x * sc, v.y * sc, v.z * sc, v.w * sc};
            __half hi[4], lo[4];
            float shi = 0.f, slo = 0.f;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                hi[q] = __float2half_rn(e[q]);
                float hf = __half2float(hi[q]);
                lo[q] = __float2half_rn(e[q] - hf);
                shi += hf;
                slo += __half2float(lo[q]);
            }
            if (on) {
                // kk = 4f.. inside the phase: block = kk/32, j = (kk/16)&1, slot = kk%16
                int kk = 4 * f, blk = kk >> 5, jj = (kk >> 4) & 1, slot = kk & 15;
                int tt0 = (slot & 7) >> 1, up = slot >> 3;   // elements 0,1 -> thread tt0, elements 2,3 -> tt0+1
                __half2* dst = reinterpret_cast<__half2*>(xs + ((size_t)blk * ncols + 2 * m) * 4);
                // uint4 of lane t holds halves [j0: k 2t,2t+1 | j0: k 2t+8,2t+9 | j1: ... | j1: ...]
                int w0 = tt0 * 4 + jj * 2 + up, w1 = (tt0 + 1) * 4 + jj * 2 + up;
                dst[w0] = __halves2half2(hi[0], hi[1]);
                dst[w1] = __halves2half2(hi[2], hi[3]);
                dst[16 + w0] = __halves2half2(lo[0], lo[1]);   // next column (lo) is 4 uint4 = 16 half2 further
                dst[16 + w1] = __halves2half2(lo[2], lo[3]);
            }
            if (SUBN) {
                // 8 consecutive lanes cover one 32-block of one row: reduce their sums
#pragma unroll
                for (int o = 1; o < 8; o <<= 1) {
                    shi += __shfl_xor_sync(0xFFFFFFFFu, shi, o);
                    slo += __shfl_xor_sync(0xFFFFFFFFu, slo, o);
                }
                if (on && (lane & 7) == 0) {
                    int blk = (4 * f) >> 5;
                    const float k8 = -8.f * 5.9604644775390625e-8f;      // -8 * 2^-24
                    float ch = k8 * shi, cl = k8 * slo;
                    cs[((size_t)blk * MT + (m >> 2)) * 4 + (m & 3)] = make_float4(ch, cl, 16.f * ch, 16.f * cl);
                }
            }
        }
        __syncthreads();

        // ---- stream this warp's chunks
        float pacc[2][MT][2];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int b = 0; b < MT; ++b) pacc[a][b][0] = pacc[a][b][1] = 0.f;

        for (int c0 = ph0 + warp; c0 < ph1; c0 += Q4_WARPS * Q4_PF) {
#pragma unroll
            for (int s = 0; s < Q4_PF; ++s) {
                const int c = c0 + s * Q4_WARPS;
                if (c < ph1) {
                    uint4 w0 = wq[s][0], w1 = wq[s][1], sv = sq[s];
                    const int cn = c + Q4_WARPS * Q4_PF;
                    if (cn < ph1) {
                        wq[s][0] = ldg_stream(wbase + (size_t)cn * Q4_UNIT_U4);
                        wq[s][1] = ldg_stream(wbase + (size_t)cn * Q4_UNIT_U4 + 32);
                        sq[s] = ldg_stream(sbase + (size_t)cn * Q4_UNIT_U4);
                    }
                    const int lb = (c - ph0) * 2;
                    uint4 bf[MT][2];
                    float4 cf[MT][2];
#pragma unroll
                    for (int bt = 0; bt < MT; ++bt)
#pragma unroll
                        for (int b = 0; b < 2; ++b) {
                            int col = bt * 8 + g;
                            bf[bt][b] = (col < ncols) ? xs[((size_t)(lb + b) * ncols + col) * 4 + t] : make_uint4(0, 0, 0, 0);
                            cf[bt][b] = SUBN ? cs[((size_t)(lb + b) * MT + bt) * 4 + t] : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    const uint32_t wt[2][4] = {{w0.x, w0.y, w0.z, w0.w}, {w1.x, w1.y, w1.z, w1.w}};
                    const uint32_t st[2][2] = {{sv.x, sv.y}, {sv.z, sv.w}};
#pragma unroll
                    for (int tile = 0; tile < 2; ++tile) {
                        float2 sA = __half22float2(*reinterpret_cast<const __half2*>(&st[tile][0]));   // row g:   block 0, 1
                        float2 sB = __half22float2(*reinterpret_cast<const __half2*>(&st[tile][1]));   // row g+8: block 0, 1
#pragma unroll
                        for (int b = 0; b < 2; ++b) {
                            uint32_t a0[4], a1[4];
                            q4_unpack<SUBN>(wt[tile][2 * b], a0);
                            q4_unpack<SUBN>(wt[tile][2 * b + 1], a1);
                            float sa = b ? sA.y : sA.x, sb = b ? sB.y : sB.x;
#pragma unroll
                            for (int bt = 0; bt < MT; ++bt) {
                                float d[4];
                                mma16816(d, a0, bf[bt][b].x, bf[bt][b].y, cf[bt][b].x, cf[bt][b].y, cf[bt][b].z, cf[bt][b].w);
                                mma16816(d, a1, bf[bt][b].z, bf[bt][b].w, d[0], d[1], d[2], d[3]);
                                pacc[tile][bt][0] = fmaf(sa, d[0] + d[1], pacc[tile][bt][0]);
                                pacc[tile][bt][1] = fmaf(sb, d[2] + d[3], pacc[tile][bt][1]);
                            }
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int b = 0; b < MT; ++b) {
                acc[a][b][0] = fmaf(pacc[a][b][0], inv_sc, acc[a][b][0]);
                acc[a][b][1] = fmaf(pacc[a][b][1], inv_sc, acc[a][b][1]);
            }
    }
    if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- reduce the 8 warps (fixed order), then the cluster's K splits (fixed order)
    const float fA = SUBN ? 16777216.f : 1.f;     // 2^24
    const float fB = SUBN ? 1048576.f : 1.f;      // 2^20 (rows g+8 carry an extra factor 16)
#pragma unroll
    for (int tile = 0; tile < 2; ++tile)
#pragma unroll
        for (int bt = 0; bt < MT; ++bt) {
            // red[w][j][r]: j = m (4*bt + t), r = row inside the pair-tile
            red[warp][4 * bt + t][tile * 16 + g] = acc[tile][bt][0] * fA;
            red[warp][4 * bt + t][tile * 16 + g + 8] = acc[tile][bt][1] * fB;
        }
    __syncthreads();
    for (int i = tid; i < 4 * MT * 32; i += Q4_THREADS) {
        int m = i >> 5, r = i & 31;
        float s = red[0][m][r];
#pragma unroll
        for (int w = 1; w < Q4_WARPS; ++w) s += red[w][m][r];
        part[m][r] = s;
    }
    if (p.splits > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        if (cluster.block_rank() == 0) {
            for (int i = tid; i < 4 * MT * 32; i += Q4_THREADS) {
                int m = i >> 5, r = i & 31;
                float s = part[m][r];
                for (int q = 1; q < p.splits; ++q) s += cluster.map_shared_rank(&part[0][0], q)[i];
                int64_t n = (int64_t)blockIdx.x * 32 + r;
                if (m < M && n < p.N) p.Y[(size_t)m * p.ldy + n] = s;
            }
        }
        cluster.sync();
    } else {
        __syncthreads();
        for (int i = tid; i < 4 * MT * 32; i += Q4_THREADS) {
            int m = i >> 5, r = i & 31;
            int64_t n = (int64_t)blockIdx.x * 32 + r;
            if (m < M && n < p.N) p.Y[(size_t)m * p.ldy + n] = part[m][r];
        }
    }
}


// ---------------------------------------------------------------------------
// the streaming kernel: M <= 4, whole x resident in shared memory
// ---------------------------------------------------------------------------
// One CTA of sixteen warps per SM and launch, no CTA-wide synchronisation
// between staging the activation and draining the runs.
//
// The unit stream is cut into contiguous runs of GROUPS (G consecutive chunks
// of one row pair-tile; the layout pads K so that a group never straddles a
// tile), one run per warp.  When the matrix has at least about one row
// pair-tile per SM, each CTA takes WHOLE tiles and its warps split them, so no
// tile is shared between CTAs; otherwise (few rows, e.g. a tensor-parallel
// shard) all warps of the grid take equal runs and tiles cut by a CTA boundary
// are finished through global scratch.  Each warp owns a private ring of
// shared-memory stages that its lane 0 keeps full with cp.async.bulk copies
// (mbarrier complete_tx), so the HBM stream of a warp never waits for its
// arithmetic and -- because the first copies are issued BEFORE
// griddepcontrol.wait -- not for the previous kernel in the stream either.
// A row pair-tile that lies wholly inside one warp's run is written straight
// to y.  A tile shared by warps of one CTA is summed through shared memory, in
// warp order, when the CTA has drained its runs.  A tile cut by the boundary
// between two CTAs is finished through global scratch (q4s_cross_cta).
constexpr int Q4S_WARPS = 16;                    // one CTA of sixteen warps per SM
constexpr int Q4S_THREADS = Q4S_WARPS * 32;
constexpr int Q4S_MAX_DEPTH = 8;                 // most ring stages per warp
constexpr int Q4_GROUP_PAD = 4;                  // chunks per row pair-tile are padded to a multiple of this
constexpr uint32_t Q4S_SPIN_LIMIT = 1u << 22;    // polls of one mbarrier before giving up
constexpr size_t Q4S_SLOT_BYTES_PER_CTA = 2 * 32 * 4 * sizeof(uint2);   // two tagged partial tiles per CTA

struct Q4StreamLaunch {
    const uint4* stream;
    const float* X;         // [M][K]; with swiglu: [M][2K] = [gate | up], and the activation is silu(gate) * up
    float* Y;               // [M][ldy]
    int M, N, K;
    int swiglu;             // 1: SwiGLU is applied while the activation is staged
    int64_t ldy;
    int nchunks;            // per row pair-tile, a multiple of G
    int groups;             // nrp * nchunks / G
    int warps_total;        // W: warps that own a run (<= NW*gridDim.x, <= groups); split mode only
    int tile_mode;          // 1: CTA b owns row pair-tiles [b*nrp/grid, (b+1)*nrp/grid) and its warps split them
    int nrp;                // row pair-tiles
    int depth;              // ring stages per warp (<= Q4S_MAX_DEPTH)
    int pre;                // stages copied before the dependency on the previous kernel resolves (the rest after the activation loads)
    uint2* partials;        // [CTAs][2][32 lanes][4] (value, tag) pairs
    int* status;            // set non-zero when a bounded wait ran out
    // row-parallel mode (xworld > 0): finished tiles are not written to Y but pushed, as (value, 1) pairs,
    // into slot [xrank] of every rank's exchange buffer; then every rank adds the xworld slots of its own
    // buffer, in rank order, into Y and clears them.  Consecutive launches alternate between the two
    // halves of the buffer, so a fast rank cannot overwrite what a slow rank has not read yet.
    int xworld, xrank;
    uint2* xpeer[8];        // rank r's exchange buffer (this rank's own for r == xrank), already offset to this launch's half
    uint2* xmine;           // == xpeer[xrank] (a separate field: the array is only ever indexed by constants, which
                            // keeps the parameter block out of local memory)
    int64_t xslot;          // uint2 per slot (>= M * N)
    uint32_t xlimit;        // polls of one element before giving up
#ifdef MPQ_TRACE
    unsigned long long* trace;   // [CTAs][16]: %globaltimer stamps of thread 0, then warp 0's cycle counts (diagnostic build only)
#endif
};

// Diagnostic build (-DMPQ_TRACE): thread 0 of every CTA records when it passed each phase of the kernel.
#ifdef MPQ_TRACE
#define Q4S_TRACE(slot)                                                        \
    if (p.trace && tid == 0) {                                                 \
        unsigned long long t_;                                                 \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                 \
        p.trace[(size_t)blockIdx.x * 16 + (slot)] = t_;                        \
    }
#define Q4S_CYC(var) long long var = clock64();
#define Q4S_CYC_ADD(acc, since) acc += clock64() - (since);
#else
#define Q4S_TRACE(slot)
#define Q4S_CYC(var)
#define Q4S_CYC_ADD(acc, since)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// 16-byte load from a 32-bit shared-memory address (half the address registers of a generic pointer)
__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// bounded wait on a phase parity: returns false when the limit ran out (the caller records it and leaves)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .u32 n;\n\t"
        "mov.u32 n, 0;\n\t"
        "WAIT_LOOP:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "@p bra WAIT_DONE;\n\t"
        "add.u32 n, n, 1;\n\t"
        "setp.lt.u32 p, n, %3;\n\t"
        "@p bra WAIT_LOOP;\n\t"
        "mov.u32 %0, 0;\n\t"
        "bra WAIT_END;\n\t"
        "WAIT_DONE:\n\t"
        "mov.u32 %0, 1;\n\t"
        "WAIT_END:\n\t"
        "}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(limit) : "memory");
    return ok != 0;
}
// Weights are read once per call: the copies carry an evict-first L2 policy so that they do not push the
// (small, re-read) activations and outputs out of L2.
__device__ __forceinline__ uint64_t l2_evict_first_policy()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t policy)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}

// floor(i * groups / W); 64-bit division costs a hundred-odd instructions, and these run before a CTA's first copy,
// so the product is divided in 32 bits whenever it fits (it does for every matrix up to a few GB)
__device__ __forceinline__ int q4s_run_start(int i, int groups, int W)
{
    const uint64_t prod = (uint64_t)(uint32_t)i * (uint32_t)groups;
    if (prod < 0x100000000ull) return (int)((uint32_t)prod / (uint32_t)W);
    return (int)(prod / (uint64_t)W);
}
// index of the warp whose run contains group gidx
__device__ __forceinline__ int q4s_owner(int gidx, int groups, int W)
{
    int i = (int)(((int64_t)gidx * W) / groups);
    while (i + 1 < W && q4s_run_start(i + 1, groups, W) <= gidx) ++i;
    while (i > 0 && q4s_run_start(i, groups, W) > gidx) --i;
    return i;
}

// A (value, tag) pair travels as ONE 64-bit access: single-copy atomic under the PTX memory model, so a
// reader that sees the tag sees the value.  (A .v2.u32 access would be two scalar accesses of unspecified order.)
__device__ __forceinline__ uint64_t pack_tagged(float v, uint32_t tag) { return ((uint64_t)tag << 32) | __float_as_uint(v); }
__device__ __forceinline__ uint2 unpack_tagged(uint64_t w) { return make_uint2((uint32_t)w, (uint32_t)(w >> 32)); }
__device__ __forceinline__ void st_tagged(uint2* p, float v, uint32_t tag)
{
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(pack_tagged(v, tag)) : "memory");
}
__device__ __forceinline__ uint2 ld_tagged(const uint2* p)
{
    uint64_t w;
    asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return unpack_tagged(w);
}
__device__ __forceinline__ void st_tagged_sys(uint2* p, float v, uint32_t tag)
{
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(pack_tagged(v, tag)) : "memory");
}
__device__ __forceinline__ uint2 ld_tagged_sys(const uint2* p)
{
    uint64_t w;
    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return unpack_tagged(w);
}

// Write one finished row pair-tile to y.  v[tile*2+h] belongs to row tile*16 + g + 8h, activation row t.
__device__ __forceinline__ void q4s_store_tile(const Q4StreamLaunch& p, const float (&v)[4], int rp, int lane)
{
    const int g = lane >> 2, t = lane & 3;
    if (t < p.M) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            int n = rp * 32 + (q >> 1) * 16 + g + 8 * (q & 1);
            if (n < p.N) {
                if (p.xworld > 0) {                      // plain peer stores over NVLink: one 8-byte store per rank
                    const size_t e = (size_t)p.xrank * p.xslot + (size_t)t * p.N + n;
#pragma unroll
                    for (int r = 0; r < 8; ++r)
                        if (r < p.xworld) st_tagged_sys(p.xpeer[r] + e, v[q], 1u);
                } else {
                    p.Y[(size_t)t * p.ldy + n] = v[q];
                }
            }
        }
    }
}

// A row pair-tile cut by the boundary between two CTAs' runs.  Every CTA but the first that shares
// the tile stores its partial as (value, 1) pairs -- one aligned 8-byte store each, so a reader that
// sees the tag sees the value, with no fence and no counter -- and carries on.  The first CTA, for
// which the tile is the END of its run, polls the others' slots (bounded), adds them in CTA order, so
// the sum does not depend on timing, writes y, and clears the slots it consumed.  A slot is written
// once and read once per launch, and the next launch writes only after this one has completed, so the
// protocol needs no per-launch state (it is safe under CUDA-graph replay).
__device__ __noinline__ void q4s_cross_cta(const Q4StreamLaunch& p, float v0, float v1, float v2, float v3, int rp, int r0,
                                           int r1, int cta_first_rp, int lane)
{
    float v[4] = {v0, v1, v2, v3};
    const int W = p.warps_total;
    const int c0 = q4s_owner(r0, p.groups, W) / Q4S_WARPS;
    if ((int)blockIdx.x != c0) {
        uint2* mine = p.partials + (((size_t)blockIdx.x * 2 + (rp == cta_first_rp ? 0 : 1)) * 32 + lane) * 4;
#pragma unroll
        for (int q = 0; q < 4; ++q) st_tagged(mine + q, v[q], 1u);
        return;
    }
    const int c1 = q4s_owner(r1 - 1, p.groups, W) / Q4S_WARPS;
    // every later CTA starts its run inside this tile, so the tile is its first one (slot 0)
    const uint2* src = p.partials + (((size_t)(c0 + 1) * 2) * 32 + lane) * 4;
    for (int c = c0 + 1; c <= c1; c += 4) {                // four contributors' loads in flight at a time
        uint2 r[4][4];
        bool ok = false;
        for (uint32_t spin = 0; spin < Q4S_SPIN_LIMIT && !ok; ++spin) {
            ok = true;
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    r[u][q] = (c + u <= c1) ? ld_tagged(src + (size_t)u * 256 + q) : make_uint2(0u, 1u);
                    ok = ok && (r[u][q].y == 1u);
                }
            ok = __all_sync(0xFFFFFFFFu, ok);
        }
        if (!ok) {
            if (lane == 0) atomicExch(p.status, 2);
            return;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                v[q] += __uint_as_float(r[u][q].x);
                if (c + u <= c1) st_tagged(const_cast<uint2*>(src) + (size_t)u * 256 + q, 0.f, 0u);   // consumed: free the slot
            }
        src += 4 * 256;
    }
    q4s_store_tile(p, v, rp, lane);
}

// One float4 of x (element index 4f of activation row m) -> normalised hi/lo fp16 fragments in xs, block
// corrections in cs.
//   xs: uint4 [chunk][2M columns][4 t][2 blocks]   column 2m = hi, 2m+1 = lo of activation row m; the uint4 of
//                                                  lane t holds halves [j0: k 2t,2t+1 | j0: k 2t+8,2t+9 | j1 ...]
//   cs: float4[chunk][M]                           (c, 16c) of block 0, (c, 16c) of block 1, c = -8 * 2^-24 * sum of
//                                                  the block's scaled x: the hi column's C operand (the lo column's is 0);
//                                                  hi + lo differs from the scaled x by < 2^-22 of it, which is what the
//                                                  sum may be off by as well
__device__ __forceinline__ void q4s_stage_one(float4 v, bool on, int m, int f, float sc, int ncols, int M, uint4* xs, float4* cs,
                                              int lane)
{
    const float e0 = v.x * sc, e1 = v.y * sc, e2 = v.z * sc, e3 = v.w * sc;
    const __half2 h01 = __floats2half2_rn(e0, e1), h23 = __floats2half2_rn(e2, e3);
    const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
    const __half2 l01 = __floats2half2_rn(e0 - f01.x, e1 - f01.y), l23 = __floats2half2_rn(e2 - f23.x, e3 - f23.y);
    float sum = (e0 + e1) + (e2 + e3);
    const int chunk = f >> 4, r = f & 15;
    const int blk = r >> 3, jj = (r >> 2) & 1, up = (r >> 1) & 1, tt0 = (r & 1) * 2;
    if (on) {
        // Column c keeps its eight 16-byte slots (t, block) at slot ^ (c & 7): the eight columns an MMA's lanes read
        // together then fall into different banks.
        __half2* dst = reinterpret_cast<__half2*>(xs + ((size_t)chunk * ncols + 2 * m) * 8);   // 8 uint4 per column
        const int s0 = tt0 * 2 + blk, s1 = s0 + 2, in = jj * 2 + up;                           // thread tt0 and tt0 + 1 of the fragment
        const int chi = (2 * m) & 7, clo = (2 * m + 1) & 7;
        dst[((s0 ^ chi) << 2) + in] = h01;
        dst[((s1 ^ chi) << 2) + in] = h23;
        dst[32 + ((s0 ^ clo) << 2) + in] = l01;           // next column (lo): 8 uint4 = 32 half2 further
        dst[32 + ((s1 ^ clo) << 2) + in] = l23;
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);   // 8 consecutive lanes cover one 32-block of one row
    if (on && (lane & 7) == 0) {
        const float c = -8.f * 5.9604644775390625e-8f * sum;                        // -8 * 2^-24
        reinterpret_cast<float2*>(cs + ((size_t)chunk * M + m))[blk] = make_float2(c, 16.f * c);
    }
}

// One pass over this thread's share of x (float4 index i = m * pk4 + f over M rows of pk4 float4): returns the largest
// |x| bit pattern seen and, if CONVERT, stages the fragments with scale sc.
template <bool CONVERT>
__device__ __forceinline__ uint32_t q4s_stage_pass(const Q4StreamLaunch& p, int pk4, int total4, float sc, int ncols, uint4* xs,
                                                   float4* cs, int tid, int lane, int threads)
{
    uint32_t mx = 0;
    const int iters = (total4 + threads - 1) / threads;
    for (int it0 = 0; it0 < iters; it0 += 4) {
        float4 v[4];
        int mm[4], ff[4];
        bool on[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {                      // up to four loads in flight per thread
            const int i = (it0 + u) * threads + tid;
            on[u] = it0 + u < iters && i < total4;
            const int ii = on[u] ? i : 0;
            mm[u] = (ii >= pk4) + (ii >= 2 * pk4) + (ii >= 3 * pk4);       // M <= 4
            ff[u] = ii - mm[u] * pk4;
            v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (on[u] && 4 * ff[u] < p.K) {
                if (p.swiglu) {
                    const float* row = p.X + (size_t)mm[u] * 2 * p.K + 4 * ff[u];
                    v[u] = swiglu_f32x4(*reinterpret_cast<const float4*>(row), *reinterpret_cast<const float4*>(row + p.K));
                } else {
                    v[u] = *reinterpret_cast<const float4*>(p.X + (size_t)mm[u] * p.K + 4 * ff[u]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if ((it0 + u) * threads >= total4) break;       // the same for the whole CTA: nothing left to stage
            mx = max(mx, __float_as_uint(v[u].x) & 0x7FFFFFFFu);
            mx = max(mx, __float_as_uint(v[u].y) & 0x7FFFFFFFu);
            mx = max(mx, __float_as_uint(v[u].z) & 0x7FFFFFFFu);
            mx = max(mx, __float_as_uint(v[u].w) & 0x7FFFFFFFu);
            if (CONVERT) q4s_stage_one(v[u], on[u], mm[u], ff[u], sc, ncols, p.M, xs, cs, lane);
        }
    }
    return mx;
}

// dynamic shared memory: ring [16 warps][depth][G units] | xs | cs | mbarriers | wpart (the warps' parked partial tiles)
template <int G>
__global__ void __launch_bounds__(Q4S_THREADS, 1) q4_stream_kernel(const __grid_constant__ Q4StreamLaunch p)
{
    constexpr int STAGE_BYTES = G * Q4_UNIT_BYTES;
    constexpr int NW = Q4S_WARPS, THREADS = Q4S_THREADS;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ uint32_t s_max[NW];
    __shared__ int wrp[NW][2];                    // the tile index of each warp's parked partial tiles, -1 if none
    __shared__ uint4 zero_pg[2];                  // what lanes outside the 2M real columns read

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int M = p.M, ncols = 2 * M, D = p.depth;
    Q4S_TRACE(0)
    if (lane < 2) wrp[warp][lane] = -1;
    if (tid < 2) zero_pg[tid] = make_uint4(0, 0, 0, 0);
    unsigned char* ring = smem_raw + (size_t)warp * D * STAGE_BYTES;
    uint4* xs = reinterpret_cast<uint4*>(smem_raw + (size_t)NW * D * STAGE_BYTES);
    float4* cs = reinterpret_cast<float4*>(reinterpret_cast<unsigned char*>(xs) + (size_t)p.nchunks * ncols * 128);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(cs) + (size_t)p.nchunks * M * 16) + warp * Q4S_MAX_DEPTH;
    float* wpart = reinterpret_cast<float*>(bars - warp * Q4S_MAX_DEPTH + NW * Q4S_MAX_DEPTH);     // [NW][2][4][32]

    const int W = p.warps_total;
    const int gw = blockIdx.x * NW + warp;
    const int gpr = p.nchunks / G;                            // groups per row pair-tile
    int cta_gb, cta_ge, gb, ge;
    if (p.tile_mode) {
        cta_gb = q4s_run_start((int)blockIdx.x, p.nrp, (int)gridDim.x) * gpr;
        cta_ge = q4s_run_start((int)blockIdx.x + 1, p.nrp, (int)gridDim.x) * gpr;
        gb = cta_gb + q4s_run_start(warp, cta_ge - cta_gb, NW);
        ge = cta_gb + q4s_run_start(warp + 1, cta_ge - cta_gb, NW);
    } else {
        cta_gb = q4s_run_start(min(W, (int)blockIdx.x * NW), p.groups, W);
        cta_ge = q4s_run_start(min(W, (int)(blockIdx.x + 1) * NW), p.groups, W);
        gb = gw < W ? q4s_run_start(gw, p.groups, W) : 0;
        ge = gw < W ? q4s_run_start(gw + 1, p.groups, W) : 0;
    }
    const int ngroups = ge - gb;
    const unsigned char* gnext = reinterpret_cast<const unsigned char*>(p.stream) + (size_t)gb * STAGE_BYTES;
    const uint32_t ring_u32 = smem_u32(ring), bars_u32 = smem_u32(bars);
    Q4S_TRACE(1)

    if (lane == 0) {
        for (int s = 0; s < D; ++s) mbar_init(&bars[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    int issued = 0;
    const uint64_t l2pol = l2_evict_first_policy();
    // p.pre stages go out before the dependency on the previous kernel resolves, the rest of the ring right after the
    // activation loads have been issued.
    auto issue_upto = [&](int n) {
        if (lane == 0) {
            for (; issued < n; ++issued) {
                mbar_expect_tx(bars_u32 + issued * 8, STAGE_BYTES);
                bulk_g2s(ring_u32 + issued * STAGE_BYTES, gnext, STAGE_BYTES, bars_u32 + issued * 8, l2pol);
                gnext += STAGE_BYTES;
            }
        }
    };
    issue_upto(min(min(D, p.pre), ngroups));
    Q4S_TRACE(2)

    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    Q4S_TRACE(3)

    // ---- stage all of x as hi/lo fp16 B fragments, scaled by the power of two that puts the largest |x| of the
    // call in [2^14, 2^15): rows up to 2^17 times smaller than the largest keep full precision in the split.  A single
    // row is first staged unscaled, in the same pass that finds its maximum, and that is kept when the maximum lies in
    // [1, 2^15) (the split is then good to 2^-25 of it); otherwise, and for several rows, a second pass stages with the scale.
    const int pk4 = p.nchunks * 16;                       // float4 per activation row, padding included
    const int total4 = M * pk4;
    uint32_t mx = M == 1 ? q4s_stage_pass<true>(p, pk4, total4, 1.f, ncols, xs, cs, tid, lane, THREADS)
                         : q4s_stage_pass<false>(p, pk4, total4, 1.f, ncols, xs, cs, tid, lane, THREADS);
    issue_upto(min(D, ngroups));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    if (lane == 0) s_max[warp] = mx;
    __syncthreads();
    mx = s_max[0];
#pragma unroll
    for (int w = 1; w < NW; ++w) mx = max(mx, s_max[w]);
    float inv_sc = 1.f;
    if (M > 1 || (mx != 0 && (mx < 0x3F800000u || mx >= 0x47000000u))) {      // 1.0, 2^15
        int emax = (int)(mx >> 23);
        float sc = 1.f;
        if (mx != 0 && emax < 255) {
            emax = max(emax, 16);
            sc = __uint_as_float((uint32_t)(268 - emax) << 23);
            inv_sc = __uint_as_float((uint32_t)(emax - 14) << 23);
        }
        q4s_stage_pass<true>(p, pk4, total4, sc, ncols, xs, cs, tid, lane, THREADS);
        __syncthreads();
    }
    Q4S_TRACE(4)

    // ---- stream this warp's run
    const float fA = 16777216.f * inv_sc;                     // 2^24: undo the subnormal weight encoding
    const float fB = 1048576.f * inv_sc;                      // 2^20: rows g+8 carry an extra factor 16
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    int rp = gb / gpr;
    int cg = gb - rp * gpr;                                   // group index inside the tile
    const int first_rp = rp;
    // per-lane shared-memory addresses into the staged activation; lanes outside the real columns sit on a page of zeros
    const bool bvalid = g < ncols, cvalid = t < M;
    const uint32_t zero_u32 = smem_u32(zero_pg);
    const uint32_t xs0 = bvalid ? smem_u32(xs) + g * 128 : zero_u32;                     // column g
    const uint32_t xb0 = bvalid ? ((2 * t) ^ g) * 16 : 0, xb1 = bvalid ? ((2 * t + 1) ^ g) * 16 : 16;   // its slots (t, block 0 / 1)
    const uint32_t cs0 = cvalid ? smem_u32(cs) + t * 16 : zero_u32;
    const uint32_t xstep = bvalid ? ncols * 128 : 0;          // bytes per chunk
    const uint32_t cstep = cvalid ? M * 16 : 0;
    uint32_t xsp = xs0 + cg * G * xstep;
    uint32_t csp = cs0 + cg * G * cstep;
    const uint32_t wlane = ring_u32 + lane * 16, slane = ring_u32 + 1024 + g * 16;
    int s = 0;
    uint32_t parity = 0;

    // a tile wholly inside this warp's run goes straight to y; a tile it shares (at most its first and its last) is parked
    auto flush = [&](int tile_rp) {
        float v[4] = {acc[0][0] * fA, acc[0][1] * fB, acc[1][0] * fA, acc[1][1] * fB};
        const int r0 = tile_rp * gpr;
        if (gb <= r0 && r0 + gpr <= ge) {
            q4s_store_tile(p, v, tile_rp, lane);
        } else {
            const int slot = tile_rp == first_rp ? 0 : 1;
#pragma unroll
            for (int q = 0; q < 4; ++q) wpart[((warp * 2 + slot) * 4 + q) * 32 + lane] = v[q];
            if (lane == 0) wrp[warp][slot] = tile_rp;
        }
    };
    bool timed_out = false;
#ifdef MPQ_TRACE
    long long cyc_wait = 0, cyc_refill = 0, cyc_first = 0;
    const long long cyc_loop0 = clock64();
#endif

    for (int j = 0; j < ngroups; ++j) {
        Q4S_CYC(c_w)
        const bool arrived = mbar_wait(bars_u32 + s * 8, parity, Q4S_SPIN_LIMIT);
        Q4S_CYC_ADD(cyc_wait, c_w)
        if (!arrived) {
            // Record it, issue nothing more, and give every copy still in flight the same generous bounded wait, so
            // that none lands in shared memory after this CTA has left (if one still does not arrive, the hazard stays).
            if (lane == 0) {
                atomicExch(p.status, 1);
                for (int idx = j + 1; idx < issued; ++idx) mbar_wait(bars_u32 + (idx % D) * 8, (uint32_t)(idx / D) & 1u, Q4S_SPIN_LIMIT);
            }
            timed_out = true;
            break;
        }
        const uint32_t st = s * STAGE_BYTES;
#pragma unroll
        for (int q = 0; q < G; ++q) {
            const uint4 w0 = lds128(wlane + st + q * Q4_UNIT_BYTES), w1 = lds128(wlane + st + q * Q4_UNIT_BYTES + 512);
            const uint4 sv = lds128(slane + st + q * Q4_UNIT_BYTES);
            const uint4 bf[2] = {lds128(xsp + xb0), lds128(xsp + xb1)};
            const uint4 cfu = lds128(csp);
            const float4 cf = make_float4(__uint_as_float(cfu.x), __uint_as_float(cfu.y), __uint_as_float(cfu.z), __uint_as_float(cfu.w));
            xsp += xstep;
            csp += cstep;
            const uint32_t wt[2][4] = {{w0.x, w0.y, w0.z, w0.w}, {w1.x, w1.y, w1.z, w1.w}};
            const uint32_t sw[2][2] = {{sv.x, sv.y}, {sv.z, sv.w}};
#pragma unroll
            for (int tile = 0; tile < 2; ++tile) {
                const float2 sA = __half22float2(*reinterpret_cast<const __half2*>(&sw[tile][0]));
                const float2 sB = __half22float2(*reinterpret_cast<const __half2*>(&sw[tile][1]));
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    uint32_t a0[4], a1[4];
                    q4_unpack<true>(wt[tile][2 * b], a0);
                    q4_unpack<true>(wt[tile][2 * b + 1], a1);
                    float d[4];
                    mma16816(d, a0, bf[b].x, bf[b].y, b ? cf.z : cf.x, 0.f, b ? cf.w : cf.y, 0.f);
                    mma16816(d, a1, bf[b].z, bf[b].w, d[0], d[1], d[2], d[3]);
                    acc[tile][0] = fmaf(b ? sA.y : sA.x, d[0] + d[1], acc[tile][0]);
                    acc[tile][1] = fmaf(b ? sB.y : sB.x, d[2] + d[3], acc[tile][1]);
                }
            }
        }
        ++cg;
        Q4S_CYC(c_r)
        __syncwarp();
        if (lane == 0 && issued < ngroups) {               // refill the stage just drained
            mbar_expect_tx(bars_u32 + s * 8, STAGE_BYTES);
            bulk_g2s(ring_u32 + s * STAGE_BYTES, gnext, STAGE_BYTES, bars_u32 + s * 8, l2pol);
            gnext += STAGE_BYTES;
            ++issued;
        }
        __syncwarp();
        Q4S_CYC_ADD(cyc_refill, c_r)
#ifdef MPQ_TRACE
        if (j == 0) cyc_first = clock64() - cyc_loop0;
#endif
        if (cg == gpr) {                                   // row pair-tile finished
            flush(rp);
            acc[0][0] = acc[0][1] = acc[1][0] = acc[1][1] = 0.f;
            cg = 0;
            ++rp;
            xsp = xs0;
            csp = cs0;
        }
        if (++s == D) { s = 0; parity ^= 1u; }
    }
    if (cg != 0 && !timed_out) flush(rp);  // the run ended inside a row pair-tile
#ifdef MPQ_TRACE
    if (p.trace && tid == 0) {
        unsigned long long* tr = p.trace + (size_t)blockIdx.x * 16;
        tr[8] = (unsigned long long)(clock64() - cyc_loop0); tr[9] = (unsigned long long)cyc_wait; tr[10] = (unsigned long long)cyc_refill;
        tr[11] = (unsigned long long)ngroups; tr[12] = (unsigned long long)cyc_first;
    }
#endif
    Q4S_TRACE(5)
    __syncthreads();
    Q4S_TRACE(6)

    // ---- tiles shared between warps: add the parked partials in warp order.  Segment (w, slot) opens a
    // tile if the valid segment before it belongs to another tile; its warp then sums the following ones.
    const int cta_first_rp = cta_gb / gpr;
    const int entry = wrp[lane >> 1][lane & 1];             // lane i holds segment i = (warp i/2, slot i%2)
#pragma unroll
    for (int slot = 0; slot < 2; ++slot) {
        const int idx0 = warp * 2 + slot;
        const int my = __shfl_sync(0xFFFFFFFFu, entry, idx0);
        if (my < 0) continue;
        uint32_t same = __ballot_sync(0xFFFFFFFFu, entry == my);
        if (same & ((1u << idx0) - 1u)) continue;           // an earlier warp opened this tile
        float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
        for (; same; same &= same - 1u) {                   // ascending segment order: a fixed summation order
            const int idx = __ffs(same) - 1;
            const float* src = wpart + (size_t)idx * 128 + lane;
            v0 += src[0]; v1 += src[32]; v2 += src[64]; v3 += src[96];
        }
        const int r0 = my * gpr, r1 = r0 + gpr;
        if (cta_gb <= r0 && r1 <= cta_ge) {
            const float v[4] = {v0, v1, v2, v3};
            q4s_store_tile(p, v, my, lane);
        } else {
            q4s_cross_cta(p, v0, v1, v2, v3, my, r0, r1, cta_first_rp, lane);
        }
    }

    Q4S_TRACE(7)

    // ---- row-parallel: add the ranks' partial outputs.  The tagged pairs need no flag and no grid
    // barrier: an element is ready when all xworld copies of it carry the tag.
    if (p.xworld > 0) {
        const uint2* mine = p.xmine;
        const int total = p.M * p.N;
        for (int e = blockIdx.x * THREADS + tid; e < total; e += gridDim.x * THREADS) {
            float sum = 0.f;
            bool ok = true;
            for (int r = 0; r < p.xworld && ok; ++r) {
                const uint2* src = mine + (size_t)r * p.xslot + e;
                uint2 v = ld_tagged_sys(src);
                for (uint32_t spin = 0; v.y != 1u && spin < p.xlimit; ++spin) {
                    __nanosleep(64);
                    v = ld_tagged_sys(src);
                }
                ok = v.y == 1u;
                sum += __uint_as_float(v.x);
                if (ok) st_tagged_sys(const_cast<uint2*>(src), 0.f, 0u);      // consumed: free the slot
            }
            if (!ok) { atomicExch(p.status, 7); break; }       // a peer never delivered: report it and leave
            const int m = e / p.N;
            p.Y[(size_t)m * p.ldy + (e - m * p.N)] = sum;
        }
    }
}

}  // namespace mpq
