// Q4 linear for up to 16 activation rows with the weights read ONCE: the "rectangle" kernel.
//
// The streaming kernel (q4.cuh) keeps the whole activation resident in shared memory, which caps it at four
// rows (and at K of a few ten thousand).  Here the matrix is cut into rectangles of whole row pair-tiles by a
// K SLICE short enough that the slice of all (up to 16) activation rows fits in shared memory as MMA-ready
// fragments; one CTA per rectangle.  Inside its rectangle a CTA works like the streaming kernel: sixteen warps
// take contiguous runs of bulk-copy groups (two chunks of one tile), each warp keeps a private ring of
// shared-memory stages full with cp.async.bulk, the weight fragments are formed once per unit and used for
// every 8-column MMA tile of the activation (MT of them, four rows each, hi and lo fp16 parts in adjacent
// columns), and tiles shared by warps are summed through shared memory in warp order.  With more than one K
// slice every rectangle writes its partial outputs to a [slice][M][N] scratch array and a second small kernel
// adds the slices in a fixed order; with one slice the outputs go straight to y.  (Adding the slices inside the
// kernel through tagged slots, as the streaming kernel does for tiles cut between CTAs, was built and measured:
// 8-byte slots double the scratch traffic and the CTAs of a tile group wait for their slowest member, which
// cost more than the second launch -- 109 against 99 us for a 7B layer at 16 rows.)  Arithmetic, layout and
// rounding are those of the streaming kernel (q4.cuh), so both give the same accuracy.
#pragma once
#include "q4.cuh"

namespace mpq {

constexpr int Q4R_WARPS = 16;
constexpr int Q4R_THREADS = Q4R_WARPS * 32;
constexpr int Q4R_G = 2;                                  // chunks per bulk copy
constexpr int Q4R_STAGE_BYTES = Q4R_G * Q4_UNIT_BYTES;
constexpr int Q4R_CACHE = 8;                              // float4 of the activation slice a thread keeps in registers while it is staged

struct Q4RectLaunch {
    const uint4* stream;
    const float* X;         // [M][K]
    float* Y;               // [M][ldy], written directly when nks == 1
    float* partial;         // [nks][M][N] otherwise
    int M, N, K;
    int64_t ldy;
    int nchunks;            // per row pair-tile in the stream (padded)
    int nrp;                // row pair-tiles
    int ntg, nks;           // tile groups x K slices = CTAs
    int slice_chunks;       // chunks per K slice, a multiple of Q4R_G (the last slice may be shorter)
    int depth;              // ring stages per warp
    int* status;
};

// One float4 of x (element 4f of the slice, activation row m of MP staged rows) -> fragments and corrections.
//   xs: uint4 [chunk][2 MP columns][4 t][2 blocks]  as in the streaming kernel
//   cs: float2[chunk][2 blocks][MP]                 (c, 16c) per row: the hi column's C operand
__device__ __forceinline__ void q4r_stage_one(float4 v, int m, int f, float sc, int MP, uint32_t xs_u32, uint32_t cs_u32, int lane)
{
    const float e0 = v.x * sc, e1 = v.y * sc, e2 = v.z * sc, e3 = v.w * sc;
    const __half2 h01 = __floats2half2_rn(e0, e1), h23 = __floats2half2_rn(e2, e3);
    const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
    const __half2 l01 = __floats2half2_rn(e0 - f01.x, e1 - f01.y), l23 = __floats2half2_rn(e2 - f23.x, e3 - f23.y);
    float sum = (e0 + e1) + (e2 + e3);
    const int chunk = f >> 4, r = f & 15;
    const int blk = r >> 3, jj = (r >> 2) & 1, up = (r >> 1) & 1, tt0 = (r & 1) * 2;
    // column c (128 bytes) keeps its eight 16-byte slots (t, block) at slot ^ (c & 7): bank-conflict-free fragment loads
    const uint32_t col = xs_u32 + ((uint32_t)(chunk * 2 * MP + 2 * m) * 8) * 16;
    const uint32_t s0 = tt0 * 2 + blk, s1 = s0 + 2, in = (uint32_t)(jj * 2 + up) * 4;
    const uint32_t chi = (2 * m) & 7, clo = (2 * m + 1) & 7;
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(col + ((s0 ^ chi) << 4) + in), "r"(*reinterpret_cast<const uint32_t*>(&h01)) : "memory");
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(col + ((s1 ^ chi) << 4) + in), "r"(*reinterpret_cast<const uint32_t*>(&h23)) : "memory");
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(col + 128 + ((s0 ^ clo) << 4) + in), "r"(*reinterpret_cast<const uint32_t*>(&l01)) : "memory");
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(col + 128 + ((s1 ^ clo) << 4) + in), "r"(*reinterpret_cast<const uint32_t*>(&l23)) : "memory");
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);   // 8 consecutive lanes cover one 32-block of one row
    if ((lane & 7) == 0) {
        const float c = -8.f * 5.9604644775390625e-8f * sum;                        // -8 * 2^-24
        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(cs_u32 + (uint32_t)((chunk * 2 + blk) * MP + m) * 8), "f"(c), "f"(16.f * c) : "memory");
    }
}

// dynamic shared memory: ring [16 warps][depth][2 units] | xs | cs | wpart [16 warps][4 MT][32] | mbarriers
// (a warp parks the partial tile its run STARTS in in wpart; the one its run ENDS in goes to the start of its own ring,
//  which is idle by then: the 16 KB that saves lets 8 rows x K = 4096 fit in one slice, with no reduction launch)
template <int MT>
__global__ void __launch_bounds__(Q4R_THREADS, 1) q4_rect_kernel(const __grid_constant__ Q4RectLaunch p)
{
    constexpr int MP = 4 * MT, NV = 4 * MT;               // staged rows; values per lane and row pair-tile
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ uint32_t s_max[Q4R_WARPS];
    __shared__ int wrp[Q4R_WARPS][2];                     // the tile index of each warp's parked partial tiles, -1 if none

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int D = p.depth;
    if (lane < 2) wrp[warp][lane] = -1;

    // ---- this CTA's rectangle: row pair-tiles [T0, T1) x chunks [C0, C1)
    const int tg = (int)blockIdx.x % p.ntg, ks = (int)blockIdx.x / p.ntg;
    const int T0 = q4s_run_start(tg, p.nrp, p.ntg), T1 = q4s_run_start(tg + 1, p.nrp, p.ntg);
    const int C0 = ks * p.slice_chunks, C1 = min(p.nchunks, C0 + p.slice_chunks);
    const int nsl = C1 - C0;                               // chunks in this slice (a multiple of Q4R_G)
    const int gpr = nsl / Q4R_G;                           // groups per tile inside the slice
    const int cta_groups = (T1 - T0) * gpr;
    const int gb = q4s_run_start(warp, cta_groups, Q4R_WARPS), ge = q4s_run_start(warp + 1, cta_groups, Q4R_WARPS);
    const int ngroups = ge - gb;

    const uint32_t smem0 = smem_u32(smem_raw);
    const uint32_t ring_u32 = smem0 + (uint32_t)(warp * D) * Q4R_STAGE_BYTES;
    const uint32_t xs_u32 = smem0 + (uint32_t)(Q4R_WARPS * D) * Q4R_STAGE_BYTES;
    const uint32_t cs_u32 = xs_u32 + (uint32_t)p.slice_chunks * 2 * MP * 128;
    const uint32_t wpart_u32 = cs_u32 + (uint32_t)p.slice_chunks * 2 * MP * 8;
    float* wpart = reinterpret_cast<float*>(smem_raw + (wpart_u32 - smem0));
    // parked partial tile (warp w, slot): slot 0 in wpart, slot 1 at the start of warp w's ring
    auto parked = [&](int w, int slot) -> float* {
        return slot == 0 ? wpart + (size_t)w * NV * 32 : reinterpret_cast<float*>(smem_raw + (size_t)w * D * Q4R_STAGE_BYTES);
    };
    const uint32_t bars_u32 = wpart_u32 + Q4R_WARPS * NV * 32 * 4 + (uint32_t)warp * Q4S_MAX_DEPTH * 8;

    if (lane == 0) {
        for (int s = 0; s < D; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bars_u32 + s * 8), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    // producer state (lane 0): the next group to copy, as (tile, group inside the slice)
    int ptile = T0 + gb / max(gpr, 1), pgi = gb - (gb / max(gpr, 1)) * gpr, issued = 0;
    const uint64_t l2pol = l2_evict_first_policy();
    auto issue_one = [&](int stage) {
        const unsigned char* src = reinterpret_cast<const unsigned char*>(p.stream) +
                                   ((size_t)ptile * p.nchunks + C0 + (size_t)pgi * Q4R_G) * Q4_UNIT_BYTES;
        mbar_expect_tx(bars_u32 + stage * 8, Q4R_STAGE_BYTES);
        bulk_g2s(ring_u32 + stage * Q4R_STAGE_BYTES, src, Q4R_STAGE_BYTES, bars_u32 + stage * 8, l2pol);
        if (++pgi == gpr) { pgi = 0; ++ptile; }
        ++issued;
    };
    if (lane == 0)
        for (int s = 0; s < min(D, ngroups); ++s) issue_one(s);      // the weights do not depend on the previous kernel

    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- stage the slice of x (MP rows, the ones beyond M as zeros), scaled so that the largest |x| lies in [2^14, 2^15)
    const int pk4 = nsl * 16;                              // float4 per staged row in this slice
    const int total4 = MP * pk4;
    const int64_t k0 = (int64_t)C0 * 64;
    // One pass over the slice where it fits: each thread keeps its first Q4R_CACHE float4 in registers between the search
    // for the largest magnitude and the conversion, with all of their loads in flight at once (read one by one, each
    // iteration of the conversion waited for its own L2 round trip: 5 to 7 us of a 37 us kernel).
    float4 cache[Q4R_CACHE];
    uint32_t mx = 0;
#pragma unroll
    for (int it = 0; it < Q4R_CACHE; ++it) {
        const int i = it * Q4R_THREADS + tid;
        const int m = i / pk4, f = i - m * pk4;
        const int64_t k = k0 + 4 * f;
        cache[it] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < total4 && m < p.M && k < p.K) cache[it] = __ldg(reinterpret_cast<const float4*>(p.X + (size_t)m * p.K + k));
    }
#pragma unroll
    for (int it = 0; it < Q4R_CACHE; ++it) {
        mx = max(mx, __float_as_uint(cache[it].x) & 0x7FFFFFFFu);
        mx = max(mx, __float_as_uint(cache[it].y) & 0x7FFFFFFFu);
        mx = max(mx, __float_as_uint(cache[it].z) & 0x7FFFFFFFu);
        mx = max(mx, __float_as_uint(cache[it].w) & 0x7FFFFFFFu);
    }
    for (int i = Q4R_CACHE * Q4R_THREADS + tid; i < p.M * pk4; i += Q4R_THREADS) {
        const int m = i / pk4, f = i - m * pk4;
        const int64_t k = k0 + 4 * f;
        if (k < p.K) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(p.X + (size_t)m * p.K + k));
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
    for (int w = 1; w < Q4R_WARPS; ++w) mx = max(mx, s_max[w]);
    int emax = (int)(mx >> 23);
    float sc = 1.f, inv_sc = 1.f;
    if (mx != 0 && emax < 255) {
        emax = max(emax, 16);
        sc = __uint_as_float((uint32_t)(268 - emax) << 23);
        inv_sc = __uint_as_float((uint32_t)(emax - 14) << 23);
    }
#pragma unroll
    for (int it = 0; it < Q4R_CACHE; ++it) {               // total4 is a multiple of 32: whole warps stay together for the shuffles
        const int i = it * Q4R_THREADS + tid;
        if (it * Q4R_THREADS + (tid & ~31) >= total4) break;
        const int m = i / pk4, f = i - m * pk4;
        q4r_stage_one(cache[it], m, f, sc, MP, xs_u32, cs_u32, lane);
    }
    // what did not fit in the registers is read again, again Q4R_CACHE loads in flight per thread
    for (int base = Q4R_CACHE * Q4R_THREADS; base < total4; base += Q4R_CACHE * Q4R_THREADS) {
#pragma unroll
        for (int it = 0; it < Q4R_CACHE; ++it) {
            const int i = base + it * Q4R_THREADS + tid;
            const int m = i / pk4, f = i - m * pk4;
            const int64_t k = k0 + 4 * f;
            cache[it] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < total4 && m < p.M && k < p.K) cache[it] = __ldg(reinterpret_cast<const float4*>(p.X + (size_t)m * p.K + k));
        }
#pragma unroll
        for (int it = 0; it < Q4R_CACHE; ++it) {
            const int i = base + it * Q4R_THREADS + tid;
            if (base + it * Q4R_THREADS + (tid & ~31) >= total4) break;
            const int m = i / pk4, f = i - m * pk4;
            q4r_stage_one(cache[it], m, f, sc, MP, xs_u32, cs_u32, lane);
        }
    }
    __syncthreads();

    // ---- stream this warp's run
    const float fA = 16777216.f * inv_sc;                  // 2^24: undo the subnormal weight encoding
    const float fB = 1048576.f * inv_sc;                   // 2^20: rows g+8 carry an extra factor 16
    float acc[2][MT][2];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < MT; ++b) acc[a][b][0] = acc[a][b][1] = 0.f;
    int rp = T0 + gb / max(gpr, 1);
    int cg = gb - (gb / max(gpr, 1)) * gpr;                // group index inside the tile's slice
    const int first_rp = rp;
    const uint32_t xlane = xs_u32 + (uint32_t)g * 128;                    // column g of MMA tile 0 ...
    const uint32_t xb[2] = {(uint32_t)((2 * t) ^ g) * 16, (uint32_t)((2 * t + 1) ^ g) * 16};   // ... and its slots (t, block 0 / 1)
    const uint32_t clane = cs_u32 + (uint32_t)t * 8;
    const uint32_t wlane = ring_u32 + lane * 16, slane = ring_u32 + 1024 + g * 16;
    int s = 0;
    uint32_t parity = 0;
    bool timed_out = false;

    // v index = bt * 4 + tile * 2 + h: activation row 4 bt + t, weight row tile * 16 + g + 8 h
    auto emit = [&](int tile_rp) {
        const bool whole = cta_groups > 0 && gb <= (tile_rp - T0) * gpr && (tile_rp - T0 + 1) * gpr <= ge;
        const int slot = tile_rp == first_rp ? 0 : 1;
#pragma unroll
        for (int bt = 0; bt < MT; ++bt)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float v = acc[q >> 1][bt][q & 1] * ((q & 1) ? fB : fA);
                if (whole) {
                    const int m = 4 * bt + t, n = tile_rp * 32 + (q >> 1) * 16 + g + 8 * (q & 1);
                    if (m < p.M && n < p.N) {
                        if (p.nks == 1) p.Y[(size_t)m * p.ldy + n] = v;
                        else p.partial[((size_t)ks * p.M + m) * p.N + n] = v;
                    }
                } else {
                    parked(warp, slot)[(bt * 4 + q) * 32 + lane] = v;
                }
            }
        if (!whole && lane == 0) wrp[warp][slot] = tile_rp;
    };

    for (int j = 0; j < ngroups; ++j) {
        if (!mbar_wait(bars_u32 + s * 8, parity, Q4S_SPIN_LIMIT)) {
            if (lane == 0) {
                atomicExch(p.status, 11);
                for (int idx = j + 1; idx < issued; ++idx) mbar_wait(bars_u32 + (idx % D) * 8, (uint32_t)(idx / D) & 1u, Q4S_SPIN_LIMIT);
            }
            timed_out = true;
            break;
        }
        const uint32_t st = s * Q4R_STAGE_BYTES;
#pragma unroll
        for (int q = 0; q < Q4R_G; ++q) {
            const int chunk = cg * Q4R_G + q;              // chunk inside the slice
            const uint4 w0 = lds128(wlane + st + q * Q4_UNIT_BYTES), w1 = lds128(wlane + st + q * Q4_UNIT_BYTES + 512);
            const uint4 sv = lds128(slane + st + q * Q4_UNIT_BYTES);
            const uint32_t wt[2][4] = {{w0.x, w0.y, w0.z, w0.w}, {w1.x, w1.y, w1.z, w1.w}};
            const uint32_t sw[2][2] = {{sv.x, sv.y}, {sv.z, sv.w}};
            float2 sA[2], sB[2];
#pragma unroll
            for (int tile = 0; tile < 2; ++tile) {
                sA[tile] = __half22float2(*reinterpret_cast<const __half2*>(&sw[tile][0]));
                sB[tile] = __half22float2(*reinterpret_cast<const __half2*>(&sw[tile][1]));
            }
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                uint4 bf[MT];
                float2 cf[MT];
#pragma unroll
                for (int bt = 0; bt < MT; ++bt) {
                    bf[bt] = lds128(xlane + (uint32_t)(chunk * 2 * MP + bt * 8) * 128 + xb[b]);
                    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(cf[bt].x), "=f"(cf[bt].y)
                                 : "r"(clane + (uint32_t)((chunk * 2 + b) * MP + bt * 4) * 8));
                }
#pragma unroll
                for (int tile = 0; tile < 2; ++tile) {
                    uint32_t a0[4], a1[4];
                    q4_unpack<true>(wt[tile][2 * b], a0);
                    q4_unpack<true>(wt[tile][2 * b + 1], a1);
                    const float sa = b ? sA[tile].y : sA[tile].x, sb = b ? sB[tile].y : sB[tile].x;
#pragma unroll
                    for (int bt = 0; bt < MT; ++bt) {
                        float d[4];
                        mma16816(d, a0, bf[bt].x, bf[bt].y, cf[bt].x, 0.f, cf[bt].y, 0.f);
                        mma16816(d, a1, bf[bt].z, bf[bt].w, d[0], d[1], d[2], d[3]);
                        acc[tile][bt][0] = fmaf(sa, d[0] + d[1], acc[tile][bt][0]);
                        acc[tile][bt][1] = fmaf(sb, d[2] + d[3], acc[tile][bt][1]);
                    }
                }
            }
        }
        ++cg;
        __syncwarp();
        if (lane == 0 && issued < ngroups) issue_one(s);    // refill the stage just drained
        if (cg == gpr) {                                   // this tile's slice is finished
            emit(rp);
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int b = 0; b < MT; ++b) acc[a][b][0] = acc[a][b][1] = 0.f;
            cg = 0;
            ++rp;
        }
        if (++s == D) { s = 0; parity ^= 1u; }
    }
    if (cg != 0 && !timed_out) emit(rp);                   // the run ended inside a tile
    __syncthreads();

    // ---- tiles shared between warps: add the parked partials in warp order (a fixed summation order)
    const int entry = wrp[lane >> 1][lane & 1];             // lane i holds segment i = (warp i/2, slot i%2)
#pragma unroll
    for (int slot = 0; slot < 2; ++slot) {
        const int idx0 = warp * 2 + slot;
        const int my = __shfl_sync(0xFFFFFFFFu, entry, idx0);
        if (my < 0) continue;
        uint32_t same = __ballot_sync(0xFFFFFFFFu, entry == my);
        if (same & ((1u << idx0) - 1u)) continue;           // an earlier warp opened this tile
        float v[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) v[i] = 0.f;
        for (; same; same &= same - 1u) {
            const int idx = __ffs(same) - 1;
            const float* src = parked(idx >> 1, idx & 1) + lane;
#pragma unroll
            for (int i = 0; i < NV; ++i) v[i] += src[i * 32];
        }
#pragma unroll
        for (int bt = 0; bt < MT; ++bt)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int m = 4 * bt + t, n = my * 32 + (q >> 1) * 16 + g + 8 * (q & 1);
                if (m < p.M && n < p.N) {
                    if (p.nks == 1) p.Y[(size_t)m * p.ldy + n] = v[bt * 4 + q];
                    else p.partial[((size_t)ks * p.M + m) * p.N + n] = v[bt * 4 + q];
                }
            }
    }

}

// y[m][n] = sum over the K slices of partial[ks][m][n], in slice order (four columns per thread where the shapes allow)
__global__ void __launch_bounds__(256) q4_rect_reduce_kernel(const float* __restrict__ partial, int nks, int M, int N, float* __restrict__ Y,
                                                             int64_t ldy)
{
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t total = (int64_t)M * N;
    const bool vec = (N & 3) == 0 && (ldy & 3) == 0 && ((reinterpret_cast<uintptr_t>(Y) | reinterpret_cast<uintptr_t>(partial)) & 15) == 0;
    if (vec) {
        const int64_t total4 = total / 4;
        for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total4; e += (int64_t)gridDim.x * blockDim.x) {
            float4 s = __ldcs(reinterpret_cast<const float4*>(partial) + e);
            for (int k = 1; k < nks; ++k) {
                const float4 t = __ldcs(reinterpret_cast<const float4*>(partial + (size_t)k * total) + e);
                s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
            }
            const int64_t m = (4 * e) / N;
            *reinterpret_cast<float4*>(Y + m * ldy + (4 * e - m * N)) = s;
        }
        return;
    }
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        float s = partial[e];
        for (int k = 1; k < nks; ++k) s += partial[(size_t)k * total + e];
        const int64_t m = e / N;
        Y[m * ldy + (e - m * N)] = s;
    }
}

}  // namespace mpq
