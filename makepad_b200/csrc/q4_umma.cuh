// Q4 linear for 5..64 activation rows on the fifth-generation tensor cores (tcgen05), weights read ONCE.
//
//   y[m][n] = sum_k (scale[n][k/32] * code[n][k]) * x[m][k]
//
// The legacy mma.sync path (q4.cuh, q4_rect.cuh) spends tensor-pipe and FMA time per activation row: it is at
// its arithmetic limit from about eight rows.  Here the products run as tcgen05.mma.kind::f16 with the WEIGHTS as
// the M = 128 operand, read from TENSOR MEMORY, and the activation rows as the N dimension (16..64), read from
// shared memory; accumulators (fp32) live in tensor memory.  Nothing but the weight expansion is left on the
// ordinary pipes, and it does not depend on the number of activation rows.
//
// EXACTNESS.  A weight s*c (fp16 scale times 4-bit code) needs 15 significant bits, an activation 22+: both
// are split.  Per 8-byte pair of codes the expansion warps form c as exact fp16 integers, hi = fp16(s*c) and
// lo = s*c - hi (one HFMA2, exact: the remainder of an fp16 product is representable), and x arrives split as
// hi + lo fp16 after a per-row power-of-two normalisation (q4u_xstage_kernel).  Per K step of 16 the products
// hi*xhi, hi*xlo (one MMA against both activation tiles) and lo*xhi; lo*xlo is below 2^-22 of the product.
// fp32 accumulation in the tensor core, in segments (see Q4U_SEG).
//
// DATA FLOW per CTA (one per SM, persistent over work items = up to four 128-row weight groups x a K range):
//   warp 0      producer: cp.async.bulk of the weight units (the same tile stream every other Q4 kernel reads: no
//               second copy of the weights) and of the staged activation tiles (shared by the item's groups)
//   warp 1      allocates tensor memory, issues the MMAs (one thread)
//   warps 2..17 expansion, four teams of four: thread = one weight row = one tensor-memory lane; shared memory ->
//               registers -> hi/lo fp16 -> tcgen05.st into the team's A-operand stage; every Q4U_SEG chunks the same
//               warps add the accumulators (tcgen05.ld) to running fp32 sums in registers, and after the item's
//               last chunk store y
// Hand-offs are mbarriers; every wait is bounded (a wait that runs out sets the status word and every role
// leaves its loop; tensor memory is freed on every path).  No TMA load uses multicast.
#pragma once
#include <cuda_fp16.h>

#include "q4.cuh"

namespace mpq {

constexpr int Q4U_TEAMS = 4;                  // expansion teams of four warps; team t owns A-operand stage t (a power of two)
constexpr int Q4U_THREADS = 64 + Q4U_TEAMS * 128;   // producer, MMA, expansion warps
constexpr int Q4U_WSTAGES = 12;               // weight ring: stages of one (group, chunk) = 4 units (a multiple of the teams)
constexpr int Q4U_WSTAGE_BYTES = 4 * Q4_UNIT_BYTES;
constexpr int Q4U_XSTAGES = 4;                // activation ring: stages of one chunk (hi tile + lo tile)
constexpr int Q4U_SEG = 16;                   // chunks (1024 of K) accumulated inside the tensor core before the sums are drained
constexpr int Q4U_A_COL = 256;                // accumulators: columns [0, 256); A stages: [256, 512)
constexpr int Q4U_MAX_T = 4;                  // most weight groups per work item (an accumulator of 2 Mp columns each, 256 in all)
constexpr uint32_t Q4U_SPIN = 1u << 22;       // polls of one mbarrier before giving up

struct Q4ULaunch {
    const uint4* stream;          // the Q4 tile stream
    const unsigned char* XS;      // staged activations: per chunk [hi: Mp rows x 128 B | lo: Mp rows x 128 B], 128-byte swizzle
    const float* inv_sc;          // [M] what undoes the per-row normalisation
    float* Y;                     // [M][ldy] (nks == 1)
    float* partial;               // [nks][M][N] otherwise
    int M, Mp, N;                 // Mp = M rounded up to 16
    int64_t ldy;
    int nchunks, nrp;             // chunks per pair-tile in the stream, pair-tiles
    int ngroups;                  // 128-row groups = ceil(nrp / 4)
    int T;                        // groups per item
    int stack;                    // 1: one MMA multiplies the hi part with both activation tiles (accumulators of 2 Mp columns)
    int nbatches, nks;            // items = nbatches * nks
    int slice_chunks;             // chunks per K range
    int* status;
};

// ---------------------------------------------------------------------------
// activation staging: fp32 rows -> hi/lo fp16 tiles in the order the MMA's shared-memory descriptor wants
// ---------------------------------------------------------------------------
// One CTA per staged row (rows >= M are zeros).  Row m of a chunk's tile lies at (m/8)*1024 + (m%8)*128 bytes;
// inside the row the 16-byte group j (8 halves) is stored at group j ^ (m % 8) (SWIZZLE_128B, K-major).
__global__ void __launch_bounds__(256) q4u_xstage_kernel(const float* __restrict__ X, int M, int Mp, int K, int nchunks,
                                                          unsigned char* __restrict__ XS, float* __restrict__ inv_sc)
{
    __shared__ uint32_t s_max[8];
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int m = blockIdx.x, tid = threadIdx.x;
    const int n4 = nchunks * 16;                           // float4 per padded row
    const size_t tile = (size_t)Mp * 128, chunk_bytes = 2 * tile;
    const size_t row_off = (size_t)(m >> 3) * 1024 + (size_t)(m & 7) * 128;
    float sc = 1.f;
    if (m < M) {
        uint32_t mx = 0;
        for (int f = tid; 4 * f < K; f += 256) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(X + (size_t)m * K + 4 * f));
            mx = max(mx, __float_as_uint(v.x) & 0x7FFFFFFFu);
            mx = max(mx, __float_as_uint(v.y) & 0x7FFFFFFFu);
            mx = max(mx, __float_as_uint(v.z) & 0x7FFFFFFFu);
            mx = max(mx, __float_as_uint(v.w) & 0x7FFFFFFFu);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        if ((tid & 31) == 0) s_max[tid >> 5] = mx;
        __syncthreads();
        mx = s_max[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) mx = max(mx, s_max[w]);
        int emax = (int)(mx >> 23);
        float inv = 1.f;
        if (mx != 0 && emax < 255) {                       // the largest |x| of the row goes to [2^14, 2^15)
            emax = max(emax, 16);
            sc = __uint_as_float((uint32_t)(268 - emax) << 23);
            inv = __uint_as_float((uint32_t)(emax - 14) << 23);
        }
        if (tid == 0) inv_sc[m] = inv;
    }
    for (int f = tid; f < n4; f += 256) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m < M && 4 * f < K) v = __ldg(reinterpret_cast<const float4*>(X + (size_t)m * K + 4 * f));
        const float e0 = v.x * sc, e1 = v.y * sc, e2 = v.z * sc, e3 = v.w * sc;
        const __half2 h01 = __floats2half2_rn(e0, e1), h23 = __floats2half2_rn(e2, e3);
        const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
        const __half2 l01 = __floats2half2_rn(e0 - f01.x, e1 - f01.y), l23 = __floats2half2_rn(e2 - f23.x, e3 - f23.y);
        const int chunk = f >> 4, kk = (f & 15) * 4;       // element inside the chunk
        const size_t off = (size_t)chunk * chunk_bytes + row_off + (size_t)(((kk >> 3) ^ (m & 7)) << 4) + (size_t)(kk & 7) * 2;
        *reinterpret_cast<uint2*>(XS + off) = make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
        *reinterpret_cast<uint2*>(XS + off + tile) = make_uint2(*reinterpret_cast<const uint32_t*>(&l01), *reinterpret_cast<const uint32_t*>(&l23));
    }
}

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ void q4u_bar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void q4u_bar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// bounded wait on a phase parity: false when the limit ran out.  (try_wait lets the waiting warp sleep; spinning on
// test_wait instead was measured slower here: eighteen spinning warps take issue slots from the ones that work.)
__device__ __forceinline__ bool q4u_bar_wait(uint32_t bar, uint32_t parity)
{
    for (uint32_t n = 0; n < Q4U_SPIN; ++n) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void q4u_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void q4u_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void q4u_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor], kind::f16, fp32 accumulate
__device__ __forceinline__ void q4u_mma(uint32_t d, uint32_t a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}"
        ::"r"(d), "r"(a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// registers -> this warp's 32 tensor-memory lanes: thread l writes lane l, register j goes to column +j
__device__ __forceinline__ void q4u_st8(uint32_t taddr, const uint32_t (&r)[8])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void q4u_ld8(uint32_t taddr, uint32_t (&r)[8])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr) : "memory");
}
// K-major operand tile, SWIZZLE_128B: rows are 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t q4u_desc_sw128(uint32_t addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);          // start address
    d |= (uint64_t)1 << 16;                         // leading byte offset field (unused for swizzled K-major): 1
    d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset: 8 rows * 128 B
    d |= (uint64_t)1 << 46;                         // descriptor version for sm_100
    d |= (uint64_t)2 << 61;                         // SWIZZLE_128B
    return d;
}

// tcgen05.ld of four accumulator columns of this warp's 32 lanes
__device__ __forceinline__ void q4u_ld4(uint32_t taddr, uint32_t (&r)[4])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
}

// dynamic shared memory (1024-byte aligned): activation ring | weight ring | barriers
__global__ void __launch_bounds__(Q4U_THREADS, 1) q4_umma_kernel(const __grid_constant__ Q4ULaunch p)
{
    extern __shared__ unsigned char smem_dyn[];
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile int s_abort;
    const uint32_t smem0 = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t xstage_bytes = 2u * p.Mp * 128u;
    const uint32_t xring = smem0, wring = xring + Q4U_XSTAGES * xstage_bytes;     // activation tiles need the 1024-byte alignment
    const uint32_t bars = wring + Q4U_WSTAGES * Q4U_WSTAGE_BYTES;
    const uint32_t w_full = bars, w_empty = w_full + 8 * Q4U_WSTAGES, x_full = w_empty + 8 * Q4U_WSTAGES, x_empty = x_full + 8 * Q4U_XSTAGES,
                   a_full = x_empty + 8 * Q4U_XSTAGES, a_empty = a_full + 8 * Q4U_TEAMS, d_full = a_empty + 8 * Q4U_TEAMS, d_empty = d_full + 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int items = p.nbatches * p.nks;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < Q4U_WSTAGES; ++s) { q4u_bar_init(w_full + 8 * s, 1); q4u_bar_init(w_empty + 8 * s, 4); }
        for (int s = 0; s < Q4U_XSTAGES; ++s) { q4u_bar_init(x_full + 8 * s, 1); q4u_bar_init(x_empty + 8 * s, 1); }
        for (int s = 0; s < Q4U_TEAMS; ++s) { q4u_bar_init(a_full + 8 * s, 4); q4u_bar_init(a_empty + 8 * s, 1); }
        q4u_bar_init(d_full, 1);
        q4u_bar_init(d_empty, 4 * Q4U_TEAMS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    q4u_fence_before();
    __syncthreads();
    q4u_fence_after();
    const uint32_t tmem = s_tmem_base;

    asm volatile("griddepcontrol.launch_dependents;");

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            const uint64_t l2pol = l2_evict_first_policy();
            int ws = 0, xs = 0;
            uint32_t wph = 0, xph = 0;
            bool first = true;
            for (int it = blockIdx.x; it < items && !s_abort; it += gridDim.x) {
                const int batch = it % p.nbatches, ks = it / p.nbatches;
                const int g0 = batch * p.T, g1 = min(p.ngroups, g0 + p.T);
                const int C0 = ks * p.slice_chunks, C1 = min(p.nchunks, C0 + p.slice_chunks);
                for (int c = C0; c < C1 && !s_abort; ++c) {
                    // this chunk's weights for every group of the item (they do not depend on the previous kernel)
                    for (int g = g0; g < g1; ++g) {
                        if (!q4u_bar_wait(w_empty + 8 * ws, wph ^ 1u)) { atomicExch(p.status, 31); s_abort = 1; break; }
                        const int npt = min(4, p.nrp - 4 * g);           // pair-tiles of this group that exist
                        mbar_expect_tx(w_full + 8 * ws, (uint32_t)npt * Q4_UNIT_BYTES);
                        for (int q = 0; q < npt; ++q)
                            bulk_g2s(wring + ws * Q4U_WSTAGE_BYTES + q * Q4_UNIT_BYTES,
                                     reinterpret_cast<const unsigned char*>(p.stream) + ((size_t)(4 * g + q) * p.nchunks + c) * Q4_UNIT_BYTES,
                                     Q4_UNIT_BYTES, w_full + 8 * ws, l2pol);
                        if (++ws == Q4U_WSTAGES) { ws = 0; wph ^= 1u; }
                    }
                    if (s_abort) break;
                    // the staged activation of this chunk is written by the kernel before this one in the stream
                    if (first) { asm volatile("griddepcontrol.wait;" ::: "memory"); first = false; }
                    if (!q4u_bar_wait(x_empty + 8 * xs, xph ^ 1u)) { atomicExch(p.status, 32); s_abort = 1; break; }
                    mbar_expect_tx(x_full + 8 * xs, xstage_bytes);
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(xring + xs * xstage_bytes), "l"(p.XS + (size_t)c * xstage_bytes), "r"(xstage_bytes), "r"(x_full + 8 * xs) : "memory");
                    if (++xs == Q4U_XSTAGES) { xs = 0; xph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // f16 x f16 -> f32, K-major both; N = Mp (against xhi) and N = 2 Mp (against the hi tile and the lo tile behind it)
            const uint32_t idesc1 = (1u << 4) | ((uint32_t)(p.Mp >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            const uint32_t idesc2 = (1u << 4) | ((uint32_t)(p.Mp >> 2) << 17) | ((uint32_t)(128 >> 4) << 24);
            const uint32_t acc_cols = p.stack ? 2 * p.Mp : p.Mp;
            int xs = 0, seq = 0, drains = 0;
            uint32_t xph = 0;
            for (int it = blockIdx.x; it < items && !s_abort; it += gridDim.x) {
                const int batch = it % p.nbatches, ks = it / p.nbatches;
                const int g0 = batch * p.T, g1 = min(p.ngroups, g0 + p.T);
                const int C0 = ks * p.slice_chunks, C1 = min(p.nchunks, C0 + p.slice_chunks);
                for (int c = C0; c < C1 && !s_abort; ++c) {
                    const bool seg_first = (c - C0) % Q4U_SEG == 0, seg_last = (c - C0) % Q4U_SEG == Q4U_SEG - 1 || c == C1 - 1;
                    // a new segment overwrites the accumulators: the expansion warps must have drained the last one
                    if (seg_first && drains > 0 && !q4u_bar_wait(d_empty, (uint32_t)(drains - 1) & 1u)) { atomicExch(p.status, 33); s_abort = 1; break; }
                    if (!q4u_bar_wait(x_full + 8 * xs, xph)) { atomicExch(p.status, 34); s_abort = 1; break; }
                    q4u_fence_after();
                    const uint64_t bx = q4u_desc_sw128(xring + xs * xstage_bytes);     // rows [0, Mp) = xhi, [Mp, 2 Mp) = xlo
                    const uint64_t bxlo = q4u_desc_sw128(xring + xs * xstage_bytes + p.Mp * 128);
                    for (int g = g0; g < g1; ++g, ++seq) {
                        const int as = seq & (Q4U_TEAMS - 1);
                        if (!q4u_bar_wait(a_full + 8 * as, (uint32_t)(seq / Q4U_TEAMS) & 1u)) { atomicExch(p.status, 35); s_abort = 1; break; }
                        q4u_fence_after();
                        // An MMA costs about 80 cycles of tensor-pipe time whatever its N (up to 64 or so): where two accumulators
                        // of 2 Mp columns per group fit, the hi part multiplies both activation tiles in ONE instruction
                        // (columns [0, Mp) = hi*xhi + lo*xhi, [Mp, 2 Mp) = hi*xlo); else three MMAs of N = Mp share Mp columns.
                        const uint32_t d = tmem + (uint32_t)(g - g0) * acc_cols;
                        const uint32_t a = tmem + Q4U_A_COL + as * 64;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {                     // K steps of 16: +32 bytes along K = +2 in the descriptor
                            const uint32_t first = (!seg_first || j > 0) ? 1u : 0u;
                            if (p.stack) {
                                q4u_mma(d, a + j * 8, bx + 2 * j, idesc2, first);
                                q4u_mma(d, a + 32 + j * 8, bx + 2 * j, idesc1, 1u);
                            } else {
                                q4u_mma(d, a + j * 8, bx + 2 * j, idesc1, first);
                                q4u_mma(d, a + j * 8, bxlo + 2 * j, idesc1, 1u);
                                q4u_mma(d, a + 32 + j * 8, bx + 2 * j, idesc1, 1u);
                            }
                        }
                        q4u_commit(a_empty + 8 * as);                   // the A stage is free when these MMAs are done
                    }
                    if (s_abort) break;
                    q4u_commit(x_empty + 8 * xs);                       // ... and so is the activation stage
                    if (++xs == Q4U_XSTAGES) { xs = 0; xph ^= 1u; }
                    if (seg_last) { q4u_commit(d_full); ++drains; }    // the segment's sums are complete
                }
            }
        }
    } else {
        // ---------------- expansion + drain: warps 2..17 = 4 teams x 4 lane quarters ----------------
        // Team tm expands every fourth (chunk, group) stage of the CTA's sequence into A stage tm; its warp qd covers the
        // rows of pair-tile qd of the group (one row per thread = one tensor-memory lane).
        const int e = warp - 2, qd = e & 3, tm = e >> 2;
        const uint32_t lanes = (uint32_t)(qd * 32) << 16;
        const int tile = lane >> 4, h = (lane >> 3) & 1, g8 = lane & 7; // this thread's weight row inside the pair-tile = lane
        const uint32_t code_off = (uint32_t)qd * Q4_UNIT_BYTES + tile * 512 + g8 * 64;
        const uint32_t scale_off = (uint32_t)qd * Q4_UNIT_BYTES + 1024 + g8 * 16 + tile * 8 + h * 4;
        const uint32_t shA = 4 * h, shB = 4 * h + 8;
        const __half2 k1032 = __floats2half2_rn(1032.f, 1032.f);
        const int mq = p.Mp >> 2;                                       // accumulator columns this team drains, per group
        float racc[Q4U_MAX_T][16];                                      // running fp32 sums of the drained segments
#pragma unroll
        for (int g = 0; g < Q4U_MAX_T; ++g)
#pragma unroll
            for (int i = 0; i < 16; ++i) racc[g][i] = 0.f;
        int seq = 0, drains = 0;
        bool live = true, waited = false;
        for (int it = blockIdx.x; it < items && live && !s_abort; it += gridDim.x) {
            const int batch = it % p.nbatches, ks = it / p.nbatches;
            const int g0 = batch * p.T, g1 = min(p.ngroups, g0 + p.T);
            const int C0 = ks * p.slice_chunks, C1 = min(p.nchunks, C0 + p.slice_chunks);
            for (int c = C0; c < C1 && live; ++c) {
                for (int g = g0; g < g1 && live; ++g, ++seq) {
                    if ((seq & (Q4U_TEAMS - 1)) != tm) continue;        // another team's stage
                    const int ws = seq % Q4U_WSTAGES;
                    if (!q4u_bar_wait(w_full + 8 * ws, (uint32_t)(seq / Q4U_WSTAGES) & 1u)) { if (lane == 0) { atomicExch(p.status, 36); s_abort = 1; } live = false; break; }
                    const bool exists = 4 * g + qd < p.nrp;              // the last group may lack pair-tiles: they expand to zeros
                    const uint32_t base = wring + ws * Q4U_WSTAGE_BYTES;
                    uint4 seg[4];
                    uint32_t sw = 0;
                    if (exists) {
#pragma unroll
                        for (int t = 0; t < 4; ++t) seg[t] = lds128(base + code_off + t * 16);
                        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(sw) : "r"(base + scale_off));
                    } else {
#pragma unroll
                        for (int t = 0; t < 4; ++t) seg[t] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);   // code 0
                    }
                    if (!q4u_bar_wait(a_empty + 8 * tm, ((uint32_t)(seq / Q4U_TEAMS) & 1u) ^ 1u)) { if (lane == 0) { atomicExch(p.status, 37); s_abort = 1; } live = false; break; }
                    q4u_fence_after();
                    const uint32_t dst = tmem + lanes + Q4U_A_COL + tm * 64;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {                        // K steps of the chunk; steps 0, 1 are the first 32-block
                        const uint32_t s16 = j < 2 ? (sw & 0xFFFFu) : (sw >> 16);
                        const uint32_t s2u = s16 | (s16 << 16);
                        const __half2 s2 = *reinterpret_cast<const __half2*>(&s2u);
                        uint32_t hi[8], lo[8];
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            const uint32_t w = j == 0 ? seg[t].x : j == 1 ? seg[t].y : j == 2 ? seg[t].z : seg[t].w;
#pragma unroll
                            for (int u = 0; u < 2; ++u) {                // k = 16j + 2t (+8): tensor-memory column t (+4) of the step
                                const uint32_t bits = ((w >> (u ? shB : shA)) & 0x000F000Fu) | 0x64006400u;      // halves 1024 + n
                                const __half2 code = __hsub2(*reinterpret_cast<const __half2*>(&bits), k1032);  // n - 8, exact
                                const __half2 vh = __hmul2(code, s2);
                                const __half2 vl = __hfma2(code, s2, __hneg2(vh));                              // exact remainder
                                hi[t + 4 * u] = *reinterpret_cast<const uint32_t*>(&vh);
                                lo[t + 4 * u] = *reinterpret_cast<const uint32_t*>(&vl);
                            }
                        }
                        q4u_st8(dst + j * 8, hi);
                        q4u_st8(dst + 32 + j * 8, lo);
                    }
                    // The stores took every register the shared-memory loads produced as operands: the loads have
                    // completed, so the weight stage may be overwritten.  (Releasing it right after issuing the loads
                    // would let the next copy land under them.)
                    __syncwarp();
                    if (lane == 0) q4u_bar_arrive(w_empty + 8 * ws);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    q4u_fence_before();
                    __syncwarp();
                    if (lane == 0) q4u_bar_arrive(a_full + 8 * tm);
                }
                if (!live) break;
                // ---- end of a K segment: add the accumulators to the running sums (the tensor core's own accumulation
                // loses about 2^-20 of the sum per MMA, so it is kept to Q4U_SEG chunks), on the item's last one store y
                const bool seg_last = (c - C0) % Q4U_SEG == Q4U_SEG - 1 || c == C1 - 1;
                if (!seg_last) continue;
                if (!q4u_bar_wait(d_full, (uint32_t)drains & 1u)) { if (lane == 0) { atomicExch(p.status, 38); s_abort = 1; } live = false; break; }
                ++drains;
                q4u_fence_after();
#pragma unroll
                for (int gi = 0; gi < Q4U_MAX_T; ++gi) {
                    if (g0 + gi >= g1) continue;
#pragma unroll
                    for (int c4 = 0; c4 < 16; c4 += 4) {
                        if (c4 >= mq) continue;
                        uint32_t r[4], r2[4] = {0u, 0u, 0u, 0u};
                        const uint32_t acc_cols = p.stack ? 2 * p.Mp : p.Mp;
                        q4u_ld4(tmem + lanes + (uint32_t)gi * acc_cols + tm * mq + c4, r);
                        if (p.stack) q4u_ld4(tmem + lanes + (uint32_t)gi * acc_cols + p.Mp + tm * mq + c4, r2);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 4; ++i) racc[gi][c4 + i] += __uint_as_float(r[i]) + __uint_as_float(r2[i]);
                    }
                }
                q4u_fence_before();
                __syncwarp();
                if (lane == 0) q4u_bar_arrive(d_empty);                 // the next segment may overwrite the accumulators
                if (c != C1 - 1) continue;
                if (!waited) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }    // inv_sc comes from the kernel before this one
#pragma unroll
                for (int gi = 0; gi < Q4U_MAX_T; ++gi) {
                    const int n = (g0 + gi) * 128 + qd * 32 + lane;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int m = tm * mq + i;
                        if (g0 + gi < g1 && i < mq && m < p.M && n < p.N) {
                            const float v = racc[gi][i] * p.inv_sc[m];
                            if (p.nks == 1) p.Y[(size_t)m * p.ldy + n] = v;
                            else p.partial[((size_t)ks * p.M + m) * p.N + n] = v;
                        }
                        racc[gi][i] = 0.f;
                    }
                }
            }
        }
    }
    q4u_fence_before();
    __syncthreads();
    if (warp == 1) {
        q4u_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

}  // namespace mpq
