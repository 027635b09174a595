// Q4 linear for up to 64 activation rows on the fifth-generation tensor cores (tcgen05), weights read ONCE.
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
// hi*xhi, hi*xlo (one MMA against both activation tiles where the accumulator has room) and lo*xhi; lo*xlo is
// below 2^-22 of the product.  fp32 accumulation in the tensor core, in segments (see Q4U_SEG).
//
// WORK.  A batch = four consecutive weight groups of 128 rows (they share the activation tiles); the sequence of
// (batch, chunk) pairs, batch-major, is cut into equal ranges of W chunks, one per CTA, so every SM gets the same
// amount whatever the matrix shape.  A range covers pieces of one or more batches; a batch that lies in one range is
// stored to y directly, a batch cut into pieces goes through one partial slice per piece, which q4u_reduce_kernel
// adds in piece order (deterministic).
//
// DATA FLOW per CTA (one per SM).  The CTA is four independent pipelines ("teams") fed by two producer warps; team t owns a
// weight ring, an A-operand stage and an accumulator in tensor memory, and handles group t of the batch:
//   warp 0          weight producer: cp.async.bulk of the weight units into the teams' rings (the same tile stream
//                   every other Q4 kernel reads: no second copy of the weights), as far ahead as the rings allow:
//                   the bytes in flight per SM are what hides the HBM latency
//   warp 21         activation producer: cp.async.bulk of the staged activation tiles (a ring of four chunks)
//   warps 1..4      one MMA issuer per team.  A single thread issues an MMA of N <= 64 only every 45..110 cycles
//                   (measured; the instruction itself needs 8..32 cycles of tensor pipe), four issuers together
//                   reach the pipe's rate (36 cycles per MMA of N = 64)
//   warps 5..20     expansion, four warps per team: thread = one weight row = one tensor-memory lane; shared memory
//                   -> registers -> hi/lo fp16 -> tcgen05.st into the team's A stage (two halves with their own
//                   hand-offs: one is filled while the MMAs of the other run); every Q4U_SEG chunks the
//                   same warps add the team's accumulator (tcgen05.ld) to running fp32 sums (thread-local memory,
//                   touched once per segment), and after the piece's last chunk store them
// Hand-offs are mbarriers; every wait is bounded (a wait that runs out sets the status word and every role
// leaves its loop; tensor memory is freed on every path).  No TMA load uses multicast.
#pragma once
#include <cuda_fp16.h>

#include "q4.cuh"

namespace mpq {

constexpr int Q4U_TEAMS = 4;                  // pipelines per CTA (a power of two): issuer warp + four expansion warps each
constexpr int Q4U_THREADS = 32 * (2 + Q4U_TEAMS + 4 * Q4U_TEAMS);   // weight producer, issuers, expansion warps, activation producer
constexpr int Q4U_MAX_WSTAGES = 8;            // weight ring PER TEAM: at most so many stages of one (group, chunk) = 4 units
constexpr int Q4U_WSTAGE_BYTES = 4 * Q4_UNIT_BYTES;
constexpr int Q4U_XSTAGES = 4;                // activation ring: stages of one chunk (hi tile + lo tile)
constexpr int Q4U_SEG = 16;                   // chunks (1024 of K) a team accumulates inside the tensor core before its sums are drained
                                              // (measured on 8192 x 28672 at 64 rows: max error 1.4e-5 of the output rms with 16,
                                              //  2.3e-5 with 32, 3.9e-5 with 64 and more: the bound the tests hold is 2e-5)
constexpr int Q4U_A_COL = 256;                // accumulators: columns [0, 256), 64 per team; A stages: [256, 512), 64 per team
constexpr uint32_t Q4U_SPIN = 1u << 22;       // tries of one mbarrier before giving up

struct Q4ULaunch {
    const uint4* stream;          // the Q4 tile stream
    const unsigned char* XS;      // staged activations: per chunk [hi: Mp rows x 128 B | lo: Mp rows x 128 B], 128-byte swizzle
    const float* inv_sc;          // [M] what undoes the per-row normalisation
    float* Y;                     // [M][ldy]: batches that lie in one CTA's range
    float* partial;               // [pieces][M][N]: batches cut into pieces
    int M, Mp, N;                 // Mp = M rounded up to 16
    int64_t ldy;
    int nchunks, nrp;             // chunks per pair-tile in the stream, pair-tiles
    int ngroups;                  // 128-row groups = ceil(nrp / 4)
    int nbatches;                 // batches of four groups
    int W;                        // (batch, chunk) pairs per CTA
    int wstages;                  // stages of each team's weight ring (what shared memory allows, up to Q4U_MAX_WSTAGES)
    int stack;                    // 1: one MMA multiplies the hi part with both activation tiles (accumulator of 2 Mp columns)
    int* status;
#ifdef MPQ_TRACE
    unsigned long long* trace;    // diagnostic build: per CTA 16 counters (see the kernel)
#endif
};

// Pieces of batch b when the (batch, chunk) sequence is cut every W: the CTAs first .. last hold one piece each.
__host__ __device__ __forceinline__ void q4u_pieces(int b, int nchunks, int W, int* first, int* last)
{
    *first = (int)(((long long)b * nchunks) / W);
    *last = (int)((((long long)b + 1) * nchunks - 1) / W);
}

// ---------------------------------------------------------------------------
// activation staging: fp32 rows -> hi/lo fp16 tiles in the order the MMA's shared-memory descriptor wants
// ---------------------------------------------------------------------------
// gridDim.x = staged rows (rows >= M are zeros), gridDim.y = parts of a row.  Row m of a chunk's tile lies at (m/8)*1024 + (m%8)*128 bytes;
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
        if (tid == 0 && blockIdx.y == 0) inv_sc[m] = inv;
    }
    // gridDim.y CTAs share a row: each finds the row's largest magnitude (the row is read from L2) and converts its part
    const int per = (n4 + (int)gridDim.y - 1) / (int)gridDim.y, f0 = (int)blockIdx.y * per, f1 = min(n4, f0 + per);
    for (int f = f0 + tid; f < f1; f += 256) {
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
// one non-suspending test of a phase parity (its round trip is about 200 cycles: tests of several barriers are issued together)
__device__ __forceinline__ uint32_t q4u_bar_test(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// bounded wait on a phase parity: false when the limit ran out.  One non-suspending test first (most waits find their
// phase complete), then try_wait, which suspends the thread for a hardware-chosen time per try.  (A suspend-time hint made
// the compiler emit a nanosleep polling loop with more instructions; spinning on test_wait issues more still; none of
// the three forms changed the kernel's time.)
__device__ __forceinline__ bool q4u_bar_wait(uint32_t bar, uint32_t parity)
{
    if (q4u_bar_test(bar, parity)) return true;
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

// dynamic shared memory (1024-byte aligned): activation ring | weight rings | barriers
#ifdef MPQ_TRACE
#define Q4U_CYC(var) long long var = clock64();
#define Q4U_CYC_ADD(acc, since) acc += clock64() - (since);
#else
#define Q4U_CYC(var)
#define Q4U_CYC_ADD(acc, since)
#endif

__device__ __forceinline__ uint32_t q4u_elect_one()
{
    uint32_t pred;
    asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
    return pred;
}

__global__ void __launch_bounds__(Q4U_THREADS, 1) q4_umma_kernel(const __grid_constant__ Q4ULaunch p)
{
    extern __shared__ unsigned char smem_dyn[];
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile int s_abort;
#ifdef MPQ_TRACE
    __shared__ unsigned long long s_tr[16];
    if (threadIdx.x < 16) s_tr[threadIdx.x] = 0;
#endif
    const uint32_t smem0 = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t xstage_bytes = 2u * p.Mp * 128u;
    const uint32_t xring = smem0, wring = xring + Q4U_XSTAGES * xstage_bytes;     // activation tiles need the 1024-byte alignment
    constexpr int NW = Q4U_TEAMS * Q4U_MAX_WSTAGES;
    const int WST = p.wstages;
    const uint32_t bars = wring + Q4U_TEAMS * WST * Q4U_WSTAGE_BYTES;
    const uint32_t w_full = bars, w_empty = w_full + 8 * NW, x_full = w_empty + 8 * NW, x_empty = x_full + 8 * Q4U_XSTAGES,
                   a_full = x_empty + 8 * Q4U_XSTAGES, a_empty = a_full + 16 * Q4U_TEAMS, d_full = a_empty + 16 * Q4U_TEAMS,
                   d_empty = d_full + 8 * Q4U_TEAMS;     // a_full / a_empty: [team][half]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // this CTA's range of the (batch, chunk) sequence
    const long long total = (long long)p.nbatches * p.nchunks;
    const long long L_begin = (long long)blockIdx.x * p.W, L_end = min(total, L_begin + p.W);

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < NW; ++s) { q4u_bar_init(w_full + 8 * s, 1); q4u_bar_init(w_empty + 8 * s, 128); }      // (only Q4U_TEAMS * WST of them are used)
        for (int s = 0; s < Q4U_XSTAGES; ++s) { q4u_bar_init(x_full + 8 * s, 1); q4u_bar_init(x_empty + 8 * s, Q4U_TEAMS); }
        for (int s = 0; s < Q4U_TEAMS; ++s) {
            for (int hf = 0; hf < 2; ++hf) { q4u_bar_init(a_full + 16 * s + 8 * hf, 128); q4u_bar_init(a_empty + 16 * s + 8 * hf, 1); }
            q4u_bar_init(d_full + 8 * s, 1); q4u_bar_init(d_empty + 8 * s, 128);
        }
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
        // ---------------- weight producer: lane = (team, pair-tile), sixteen copies per instruction ----------------
        const int tm = lane >> 2, q = lane & 3;
        const uint64_t l2pol = l2_evict_first_policy();
        int wn = 0;                                      // stages loaded so far for this lane's team
        int b = (int)(L_begin / p.nchunks), c = (int)(L_begin % p.nchunks);
        for (long long L = L_begin; L < L_end && !s_abort; ++L) {
            const int g = b * Q4U_TEAMS + tm;
            const bool active = lane < 4 * Q4U_TEAMS && g < p.ngroups;
            const int ws = tm * WST + wn % WST;
            bool ok = true;
            if (active) {
                ok = q4u_bar_wait(w_empty + 8 * ws, ((uint32_t)(wn / WST) & 1u) ^ 1u);
                const int npt = min(4, p.nrp - 4 * g);               // pair-tiles of this group that exist
                if (ok && q == 0) mbar_expect_tx(w_full + 8 * ws, (uint32_t)npt * Q4_UNIT_BYTES);
                if (ok && q < npt)
                    bulk_g2s(wring + ws * Q4U_WSTAGE_BYTES + q * Q4_UNIT_BYTES,
                             reinterpret_cast<const unsigned char*>(p.stream) + ((size_t)(4 * g + q) * p.nchunks + c) * Q4_UNIT_BYTES,
                             Q4_UNIT_BYTES, w_full + 8 * ws, l2pol);
                ++wn;
            }
            if (__any_sync(0xFFFFFFFFu, !ok)) { if (lane == 0) { atomicExch(p.status, 31); s_abort = 1; } break; }
            if (++c == p.nchunks) { c = 0; ++b; }
        }
    } else if (warp == 1 + 5 * Q4U_TEAMS) {
        // ---------------- activation producer ----------------
        if (lane == 0) {
            // the staged activation is written by the kernel before this one in the stream
            asm volatile("griddepcontrol.wait;" ::: "memory");
            int sc = 0;                                  // chunks so far
            int c = (int)(L_begin % p.nchunks);
            for (long long L = L_begin; L < L_end && !s_abort; ++L, ++sc, c = c + 1 == p.nchunks ? 0 : c + 1) {
                const int xs = sc % Q4U_XSTAGES;
                if (!q4u_bar_wait(x_empty + 8 * xs, ((uint32_t)(sc / Q4U_XSTAGES) & 1u) ^ 1u)) { atomicExch(p.status, 32); s_abort = 1; break; }
                mbar_expect_tx(x_full + 8 * xs, xstage_bytes);
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(xring + xs * xstage_bytes), "l"(p.XS + (size_t)c * xstage_bytes), "r"(xstage_bytes), "r"(x_full + 8 * xs) : "memory");
            }
        }
    } else if (warp <= Q4U_TEAMS) {
        // ---------------- MMA issuer of team tm: the whole warp runs the loop, one elected lane issues ----------------
        const int tm = warp - 1;
        // f16 x f16 -> f32, K-major both; N = Mp (against one activation tile) or 2 Mp (the hi tile and the lo tile behind it)
        const uint32_t idesc1 = (1u << 4) | ((uint32_t)(p.Mp >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        const uint32_t idesc2 = (1u << 4) | ((uint32_t)(p.Mp >> 2) << 17) | ((uint32_t)(128 >> 4) << 24);
        const uint32_t d = tmem + (uint32_t)tm * 64;
        const uint32_t a = tmem + Q4U_A_COL + (uint32_t)tm * 64;
        int n = 0, drains = 0, seg_n = 0, xs = 0;
        uint32_t xph = 0;
#ifdef MPQ_TRACE
        long long cyc_x = 0, cyc_a = 0, cyc_d = 0, cyc_issue = 0;
        const long long cyc_t0 = clock64();
#endif
        int b = (int)(L_begin / p.nchunks), c = (int)(L_begin % p.nchunks) - 1;
        bool live = true;
        for (long long L = L_begin; L < L_end && live; ++L) {
            if (++c == p.nchunks) { c = 0; ++b; }
            const int xs_now = xs;
            const uint32_t xph_now = xph;
            if (++xs == Q4U_XSTAGES) { xs = 0; xph ^= 1u; }
            Q4U_CYC(t_x)
            const uint32_t okx = q4u_bar_test(x_full + 8 * xs_now, xph_now);
            const uint32_t okf0 = q4u_bar_test(a_full + 16 * tm, (uint32_t)n & 1u);      // (only meaningful when this team's group exists)
            if (!okx && !q4u_bar_wait(x_full + 8 * xs_now, xph_now)) { if (lane == 0) { atomicExch(p.status, 34); s_abort = 1; } break; }
            Q4U_CYC_ADD(cyc_x, t_x)
            if (b * Q4U_TEAMS + tm >= p.ngroups) {           // the last batch may lack groups: only the activation stage's hand-back
                if (lane == 0) q4u_bar_arrive(x_empty + 8 * xs_now);
                continue;
            }
            // a new segment overwrites the accumulator: the expansion warps must have drained the last one
            Q4U_CYC(t_d)
            if (seg_n == 0 && drains > 0 && !q4u_bar_wait(d_empty + 8 * tm, (uint32_t)(drains - 1) & 1u)) { if (lane == 0) { atomicExch(p.status, 33); s_abort = 1; } break; }
            Q4U_CYC_ADD(cyc_d, t_d)
            ++seg_n;
            const bool seg_last = seg_n == Q4U_SEG || c == p.nchunks - 1 || L == L_end - 1;      // the segment, the batch or the range ends
            const uint64_t bx = q4u_desc_sw128(xring + xs_now * xstage_bytes);     // rows [0, Mp) = xhi, [Mp, 2 Mp) = xlo
            const uint64_t bxlo = q4u_desc_sw128(xring + xs_now * xstage_bytes + p.Mp * 128);
            // The A stage has two halves (K steps 0, 1 and 2, 3), each with its own hand-offs: the expansion warps fill
            // one while the MMAs of the other run.
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                Q4U_CYC(t_a)
                if (!(hf == 0 && okf0) && !q4u_bar_wait(a_full + 16 * tm + 8 * hf, (uint32_t)n & 1u)) { if (lane == 0) { atomicExch(p.status, 35); s_abort = 1; } live = false; break; }
                Q4U_CYC_ADD(cyc_a, t_a)
                q4u_fence_after();
                Q4U_CYC(t_i)
                if (q4u_elect_one()) {
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj) {              // K steps of 16: +32 bytes along K = +2 in the descriptor
                        const int j = 2 * hf + jj;
                        const uint32_t ahi = a + hf * 32 + jj * 8, alo = ahi + 16;
                        const uint32_t acc = (seg_n > 1 || j > 0) ? 1u : 0u;
                        if (p.stack) {                            // columns [0, Mp) = hi*xhi + lo*xhi, [Mp, 2 Mp) = hi*xlo
                            q4u_mma(d, ahi, bx + 2 * j, idesc2, acc);
                            q4u_mma(d, alo, bx + 2 * j, idesc1, 1u);
                        } else {
                            q4u_mma(d, ahi, bx + 2 * j, idesc1, acc);
                            q4u_mma(d, ahi, bxlo + 2 * j, idesc1, 1u);
                            q4u_mma(d, alo, bx + 2 * j, idesc1, 1u);
                        }
                    }
                    q4u_commit(a_empty + 16 * tm + 8 * hf);     // this half of the A stage is free when these MMAs are done
                    if (hf == 1) {
                        q4u_commit(x_empty + 8 * xs_now);       // ... and this team is done with the activation stage
                        if (seg_last) q4u_commit(d_full + 8 * tm);   // the segment's sums are complete
                    }
                }
                __syncwarp();
                Q4U_CYC_ADD(cyc_issue, t_i)
            }
            ++n;
            if (seg_last) { ++drains; seg_n = 0; }
        }
#ifdef MPQ_TRACE
        if (p.trace && lane == 0 && tm == 0) {
            unsigned long long* tr = p.trace + (size_t)blockIdx.x * 32;
            tr[0] = (unsigned long long)(clock64() - cyc_t0); tr[1] = (unsigned long long)cyc_x; tr[2] = (unsigned long long)cyc_d;
            tr[3] = (unsigned long long)cyc_a; tr[4] = (unsigned long long)cyc_issue; tr[5] = (unsigned long long)n;
        }
#endif
    } else {
        // ---------------- expansion + drain: warps 5..20 = 4 teams x 4 lane quarters ----------------
        // Warp qd of a team covers the rows of pair-tile qd of the team's group (one row per thread = one tensor-memory lane).
        const int e = warp - 1 - Q4U_TEAMS, qd = e & 3, tm = e >> 2;
        const uint32_t lanes = (uint32_t)(qd * 32) << 16;
        const int tile = lane >> 4, h = (lane >> 3) & 1, g8 = lane & 7; // this thread's weight row inside the pair-tile = lane
        const uint32_t code_off = (uint32_t)qd * Q4_UNIT_BYTES + tile * 512 + g8 * 64;
        const uint32_t scale_off = (uint32_t)qd * Q4_UNIT_BYTES + 1024 + g8 * 16 + tile * 8 + h * 4;
        const uint32_t shA = 4 * h, shB = 4 * h + 8;
        const uint32_t k1032 = 0x64086408u;                             // fp16 1032, twice
        const uint32_t dst = tmem + lanes + Q4U_A_COL + (uint32_t)tm * 64;
        const uint32_t dacc = tmem + lanes + (uint32_t)tm * 64;
        float racc[64];                                                 // running fp32 sums of the drained segments, one per activation row (local memory: touched once per segment)
#pragma unroll
        for (int i = 0; i < 64; ++i) racc[i] = 0.f;
        int n = 0, drains = 0, seg_n = 0, wsi = 0;
        uint32_t wph = 0;
        bool waited = false, live = true;
        float isc0 = 0.f, isc1 = 0.f;
#ifdef MPQ_TRACE
        long long cyc_w = 0, cyc_ae = 0, cyc_df = 0, cyc_exp = 0, cyc_st = 0, cyc_drain = 0, cyc_store = 0, gap_top = 0, gap_lds = 0, gap_arr = 0, t_prev = 0;
        const long long cyc_t0 = clock64();
#endif
        int b = (int)(L_begin / p.nchunks), c = (int)(L_begin % p.nchunks) - 1;
        for (long long L = L_begin; L < L_end && live; ++L) {
            if (++c == p.nchunks) { c = 0; ++b; }
            const int g = b * Q4U_TEAMS + tm;
            if (g >= p.ngroups) continue;                               // no such group in the last batch
            const bool exists = 4 * g + qd < p.nrp;                     // the last group may lack pair-tiles: they expand to zeros
            const int ws = tm * WST + wsi;
            const uint32_t wph_now = wph;
            if (++wsi == WST) { wsi = 0; wph ^= 1u; }
#ifdef MPQ_TRACE
            if (t_prev) gap_top += clock64() - t_prev;
#endif
            Q4U_CYC(t_w)
            // the stage's three waits usually find their phases complete: their tests go out together (one round trip)
            const uint32_t okw = q4u_bar_test(w_full + 8 * ws, wph_now);
            const uint32_t oka[2] = {q4u_bar_test(a_empty + 16 * tm, ((uint32_t)n & 1u) ^ 1u), q4u_bar_test(a_empty + 16 * tm + 8, ((uint32_t)n & 1u) ^ 1u)};
            if (!okw && !q4u_bar_wait(w_full + 8 * ws, wph_now)) { if (lane == 0) { atomicExch(p.status, 36); s_abort = 1; } break; }
            Q4U_CYC_ADD(cyc_w, t_w)
            Q4U_CYC(t_g1)
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
            Q4U_CYC_ADD(gap_lds, t_g1)
            // Two halves of the A stage (K steps 0, 1 = the first 32-block; 2, 3 = the second): while the MMAs of one half
            // run, the other is being filled.
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                Q4U_CYC(t_ae)
                if (!oka[hf] && !q4u_bar_wait(a_empty + 16 * tm + 8 * hf, ((uint32_t)n & 1u) ^ 1u)) { if (lane == 0) { atomicExch(p.status, 37); s_abort = 1; } live = false; break; }
                Q4U_CYC_ADD(cyc_ae, t_ae)
                q4u_fence_after();
                Q4U_CYC(t_e)
                const uint32_t s16 = hf == 0 ? (sw & 0xFFFFu) : (sw >> 16);
                const uint32_t s2u = s16 | (s16 << 16);
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    const int j = 2 * hf + jj;
                    uint32_t hi[8], lo[8];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const uint32_t w = j == 0 ? seg[t].x : j == 1 ? seg[t].y : j == 2 ? seg[t].z : seg[t].w;
#pragma unroll
                        for (int u = 0; u < 2; ++u) {            // k = 16j + 2t (+8): tensor-memory column t (+4) of the step
                            const uint32_t bits = ((w >> (u ? shB : shA)) & 0x000F000Fu) | 0x64006400u;      // halves 1024 + n
                            uint32_t code, vh, vl;                                                             // fp16 pairs in plain registers
                            asm("sub.f16x2 %0, %1, %2;" : "=r"(code) : "r"(bits), "r"(k1032));                // n - 8, exact
                            asm("mul.f16x2 %0, %1, %2;" : "=r"(vh) : "r"(code), "r"(s2u));
                            asm("{\n\t.reg .b32 t;\n\tneg.f16x2 t, %3;\n\tfma.rn.f16x2 %0, %1, %2, t;\n\t}" : "=r"(vl) : "r"(code), "r"(s2u), "r"(vh));   // exact remainder
                            hi[t + 4 * u] = vh;
                            lo[t + 4 * u] = vl;
                        }
                    }
                    q4u_st8(dst + hf * 32 + jj * 8, hi);
                    q4u_st8(dst + hf * 32 + 16 + jj * 8, lo);
                }
                Q4U_CYC_ADD(cyc_exp, t_e)
                if (hf == 1) {
                    // The stores took every register the shared-memory loads produced as operands: the loads have
                    // completed, so the weight stage may be overwritten.  (Releasing it right after issuing the loads
                    // would let the next copy land under them.)
                    q4u_bar_arrive(w_empty + 8 * ws);             // every thread, after its own stores took its registers
                }
                Q4U_CYC(t_s)
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                q4u_fence_before();
                q4u_bar_arrive(a_full + 16 * tm + 8 * hf);         // every thread, after its own stores are complete
                Q4U_CYC_ADD(cyc_st, t_s)
            }
            if (!live) break;
#ifdef MPQ_TRACE
            t_prev = clock64();
#endif
            ++n; ++seg_n;
            // ---- end of a K segment: add the accumulator to the running sums (the tensor core's own accumulation
            // loses about 2^-20 of the sum per MMA, so it is kept to Q4U_SEG chunks)
            const bool piece_last = c == p.nchunks - 1 || L == L_end - 1;
            if (!(seg_n == Q4U_SEG || piece_last)) continue;
            seg_n = 0;
            Q4U_CYC(t_df)
            if (!q4u_bar_wait(d_full + 8 * tm, (uint32_t)drains & 1u)) { if (lane == 0) { atomicExch(p.status, 38); s_abort = 1; } break; }
            Q4U_CYC_ADD(cyc_df, t_df)
            ++drains;
            q4u_fence_after();
            Q4U_CYC(t_dr)
#ifdef MPQ_TRACE
            if (p.trace && lane == 0 && e == 0 && drains <= 4) s_tr[2 * (drains - 1)] = (unsigned long long)(clock64() - cyc_t0);
#endif
            {
                // 32 accumulator columns per wait.  Columns: [0, Mp) (+ [Mp, 2 Mp) of the stacked form, which add to the same rows).
                // The block loop is not unrolled, so that racc is addressed dynamically and stays in local memory.
                const int ncols = p.stack ? 2 * p.Mp : p.Mp;
#pragma unroll 1
                for (int blk = 0; 32 * blk < ncols; ++blk) {
                    uint32_t r[32];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint32_t (&rq)[8] = *reinterpret_cast<uint32_t (*)[8]>(&r[8 * q]);
                        if (32 * blk + 8 * q < ncols) q4u_ld8(dacc + 32 * blk + 8 * q, rq);
                        else {
#pragma unroll
                            for (int i = 0; i < 8; ++i) rq[i] = 0u;
                        }
                    }
#ifdef MPQ_TRACE
                    if (p.trace && lane == 0 && e == 0 && drains == 1 && blk == 0) s_tr[11] = (unsigned long long)(clock64() - cyc_t0);
#endif
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#ifdef MPQ_TRACE
                    if (p.trace && lane == 0 && e == 0 && drains == 1 && blk == 0) s_tr[12] = (unsigned long long)(clock64() - cyc_t0);
#endif
                    if (p.stack && p.Mp == 16) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) racc[i] += __uint_as_float(r[i]) + __uint_as_float(r[16 + i]);
                    } else {
                        float* sums = racc + (p.stack ? 0 : 32 * blk);
#pragma unroll
                        for (int i = 0; i < 32; ++i) sums[i] += __uint_as_float(r[i]);
                    }
                }
            }
#ifdef MPQ_TRACE
            if (p.trace && lane == 0 && e == 0 && drains == 1) s_tr[13] = (unsigned long long)(clock64() - cyc_t0);
#endif
            q4u_fence_before();
            q4u_bar_arrive(d_empty + 8 * tm);                   // (every thread) the next segment may overwrite the accumulator
            Q4U_CYC_ADD(cyc_drain, t_dr)
#ifdef MPQ_TRACE
            if (p.trace && lane == 0 && e == 0 && drains <= 4) s_tr[1 + 2 * (drains - 1)] = (unsigned long long)(clock64() - cyc_t0);
#endif
            if (!piece_last) continue;
            Q4U_CYC(t_so)
            // ---- the piece's sums: to y when this range holds the whole batch, else to the piece's slice
            // inv_sc comes from the kernel before this one.  Lane l keeps rows l and l + 32 of it: read inside the store loop
            // the loads would be ordered behind the stores (they may alias for all the compiler knows), one round trip per row.
            if (!waited) {
                asm volatile("griddepcontrol.wait;" ::: "memory");
                waited = true;
                isc0 = lane < p.M ? p.inv_sc[lane] : 0.f;
                isc1 = lane + 32 < p.M ? p.inv_sc[lane + 32] : 0.f;
            }
            int pf, pl;
            q4u_pieces(b, p.nchunks, p.W, &pf, &pl);
            const int nrow = g * 128 + qd * 32 + lane;
            float* out = pf == pl ? p.Y : p.partial + (size_t)((int)blockIdx.x - pf) * p.M * p.N;
            const int64_t ld = pf == pl ? p.ldy : (int64_t)p.N;
#pragma unroll
            for (int m = 0; m < 64; ++m) {
                const float sc = __shfl_sync(0xFFFFFFFFu, m < 32 ? isc0 : isc1, m & 31);
                if (m < p.M && nrow < p.N) out[(size_t)m * ld + nrow] = racc[m] * sc;
                racc[m] = 0.f;
            }
            Q4U_CYC_ADD(cyc_store, t_so)
        }
#ifdef MPQ_TRACE
        if (p.trace && lane == 0 && e == 0) {
            p.trace[(size_t)blockIdx.x * 32 + 6] = (unsigned long long)cyc_store;
            p.trace[(size_t)blockIdx.x * 32 + 24] = (unsigned long long)gap_top;
            p.trace[(size_t)blockIdx.x * 32 + 25] = (unsigned long long)gap_lds;
            p.trace[(size_t)blockIdx.x * 32 + 26] = (unsigned long long)gap_arr;
            for (int i = 0; i < 8; ++i) p.trace[(size_t)blockIdx.x * 32 + 16 + i] = s_tr[i];
            for (int i = 11; i < 14; ++i) p.trace[(size_t)blockIdx.x * 32 + 16 + i] = s_tr[i];
            unsigned long long* tr = p.trace + (size_t)blockIdx.x * 32 + 8;
            tr[0] = (unsigned long long)(clock64() - cyc_t0); tr[1] = (unsigned long long)cyc_w; tr[2] = (unsigned long long)cyc_ae;
            tr[3] = (unsigned long long)cyc_exp; tr[4] = (unsigned long long)cyc_st; tr[5] = (unsigned long long)cyc_df;
            tr[6] = (unsigned long long)cyc_drain; tr[7] = (unsigned long long)n;
        }
#endif
    }
    q4u_fence_before();
    __syncthreads();
    if (warp == 1) {
        q4u_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

// y[m][n] = sum of the pieces' partial slices, in piece order, for the batches the main kernel cut into pieces.
// One thread per four consecutive columns (N is a multiple of 4 or the tail is done one by one); all rows m of them.
__global__ void __launch_bounds__(256) q4u_reduce_kernel(const float* __restrict__ partial, int M, int N, int nchunks, int W,
                                                          float* __restrict__ Y, int64_t ldy)
{
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int nq = (N + 3) / 4;
    const bool vec = (N & 3) == 0 && (ldy & 3) == 0 && ((reinterpret_cast<uintptr_t>(Y) | reinterpret_cast<uintptr_t>(partial)) & 15) == 0;
    const int64_t total = (int64_t)M * nq;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / nq), n = (int)(i % nq) * 4;
        int pf, pl;
        q4u_pieces(n / (128 * Q4U_TEAMS), nchunks, W, &pf, &pl);      // four columns never straddle a batch of 512
        if (pf == pl) continue;
        const int np = pl - pf + 1;
        if (vec) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < np; ++s) {
                const float4 t = __ldcs(reinterpret_cast<const float4*>(partial + ((size_t)s * M + m) * N + n));
                v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
            }
            *reinterpret_cast<float4*>(Y + (size_t)m * ldy + n) = v;
        } else {
            for (int k = 0; k < 4 && n + k < N; ++k) {
                float v = 0.f;
                for (int s = 0; s < np; ++s) v += partial[((size_t)s * M + m) * N + n + k];
                Y[(size_t)m * ldy + n + k] = v;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// probe: how fast can `issuers` threads (one per warp, each with its own accumulator and A columns) issue
// tcgen05.mma.kind::f16 of 128 x n_cols x 16 with A in tensor memory?  Per CTA the cycles from the first issue to the
// completion of the last MMA of warp 0 go to cycles[blockIdx.x].  Operands are constants (1.0); nothing else runs.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 1) q4u_mma_probe_kernel(int n_cols, int issuers, int reps, long long* __restrict__ cycles,
                                                                int* __restrict__ status)
{
    extern __shared__ unsigned char smem_dyn[];
    __shared__ uint32_t s_tmem_base;
    const uint32_t smem0 = (smem_u32(smem_dyn) + 1023u) & ~1023u;             // B tile: up to 64 rows x 128 bytes
    const uint32_t bars = smem0 + 8192;
    for (int i = threadIdx.x; i < 8192 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem_dyn + (smem0 - smem_u32(smem_dyn)))[i] = 0x3C003C00u;
    if (threadIdx.x == 0) {
        for (int w = 0; w < 4; ++w) q4u_bar_init(bars + 8 * w, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    q4u_fence_before();
    __syncthreads();
    q4u_fence_after();
    const uint32_t tmem = s_tmem_base;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    {
        const uint32_t ones[8] = {0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u};
        for (int c = 0; c < 128; c += 8) q4u_st8(tmem + ((uint32_t)(warp * 32) << 16) + Q4U_A_COL + c, ones);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    q4u_fence_before();
    __syncthreads();
    q4u_fence_after();
    if (warp < issuers && lane == 0) {
        const uint32_t idesc = (1u << 4) | ((uint32_t)(n_cols >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        const uint64_t bd = q4u_desc_sw128(smem0);
        const uint32_t d = tmem + (uint32_t)warp * 64, a = tmem + Q4U_A_COL + (uint32_t)warp * 32;
        const long long t0 = clock64();
        for (int r = 0; r < reps; ++r) {
#pragma unroll
            for (int j = 0; j < 4; ++j) q4u_mma(d, a + j * 8, bd + 2 * j, idesc, (r > 0 || j > 0) ? 1u : 0u);
        }
        q4u_commit(bars + 8 * warp);
        if (!q4u_bar_wait(bars + 8 * warp, 0)) atomicExch(status, 39);
        if (warp == 0) cycles[blockIdx.x] = clock64() - t0;
    }
    q4u_fence_before();
    __syncthreads();
    if (warp == 0) {
        q4u_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

}  // namespace mpq
