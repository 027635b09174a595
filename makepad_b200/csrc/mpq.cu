// libmpq: the C ABI declared in include/mpq.h.  Host-side validation, handle
// management and launch heuristics live here; the kernels are in the .cuh files.
// There is no CPU fallback anywhere in this library: every compute entry point
// launches a CUDA kernel or returns an error status.
#include "../../include/mpq.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>

#include "nvfp4.cuh"
#include "q4.cuh"

using namespace mpq;

struct mpq_context {
    uint32_t magic;
    int device;
    cudaDeviceProp prop;
    std::string err;
    int64_t launches;
    bool pdl;                 // programmatic dependent launch between consecutive linears
    int q4_variant;           // 0 = subnormal-fp16 weights (default), 1 = magic-number conversion
    // staging for the *_host convenience calls (grown on demand)
    float *hx, *hy;
    size_t hx_bytes, hy_bytes;
    // scratch of the streaming Q4 kernel: tagged partial tiles of row pair-tiles cut by a boundary
    // between two CTAs' runs (two slots per CTA; write-once / read-once per launch), one status word
    uint2* q4_partials;
    int q4_partials_warps;
    int* q4_status;
    bool q4_stream;           // use the streaming kernel where the activation fits in shared memory
    int q4_group;             // chunks per bulk copy of the streaming kernel (2 or 4)
    bool q4_tile_mode;        // let CTAs own whole row pair-tiles when the matrix has enough of them
    int q4_depth;             // most ring stages per warp
    int q4_pre;               // stages copied before the dependency resolves
    bool q4_slab4;            // M > 4 as slabs of four rows through the streaming kernel
    Nvfp4Scratch fp4;
};

struct mpq_weight {
    uint32_t magic;
    int fmt;
    int device;
    Q4Dev q4;
    Nvfp4Dev fp4;
};

struct mpq_exchange {
    uint32_t magic;
    int device, rank, world;
    int64_t max_floats;          // capacity of one slot, in values
    uint2* local;                // [2 halves][world slots][max_floats] (value, tag) pairs
    uint2* peer[8];              // every rank's buffer as mapped here (peer[rank] == local)
    bool opened[8];              // mapped with cudaIpcOpenMemHandle (to be closed on destroy)
    bool attached;
    uint32_t calls;              // launches so far: its parity picks the half of the buffer
    uint32_t wait_limit;
};

static const uint32_t CTX_MAGIC = 0x4D505143u, W_MAGIC = 0x4D505157u, X_MAGIC = 0x4D505158u;
static bool x_ok(const mpq_exchange* x) { return x && x->magic == X_MAGIC; }

static int32_t fail(mpq_context* ctx, int32_t code, const char* fmt, ...)
{
    if (ctx) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        ctx->err = buf;
    }
    return code;
}

#define CU_TRY(ctx, expr)                                                                         \
    do {                                                                                          \
        cudaError_t e__ = (expr);                                                                 \
        if (e__ != cudaSuccess)                                                                   \
            return fail(ctx, MPQ_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, __LINE__); \
    } while (0)

static bool ctx_ok(const mpq_context* c) { return c && c->magic == CTX_MAGIC; }
static bool w_ok(const mpq_weight* w) { return w && w->magic == W_MAGIC; }
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

extern "C" const char* mpq_status_string(int32_t s)
{
    switch (s) {
        case MPQ_OK: return "ok";
        case MPQ_ERR_INVALID_ARG: return "invalid argument";
        case MPQ_ERR_SHAPE: return "unsupported shape";
        case MPQ_ERR_ALIGN: return "misaligned pointer";
        case MPQ_ERR_CUDA: return "CUDA error";
        case MPQ_ERR_UNSUPPORTED: return "unsupported device or size";
        case MPQ_ERR_PEER_TIMEOUT: return "peer wait timed out";
        case MPQ_ERR_STATE: return "invalid call order";
        default: return "unknown status";
    }
}

extern "C" int32_t mpq_context_create(int32_t device, mpq_context** out)
{
    if (!out) return MPQ_ERR_INVALID_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return MPQ_ERR_CUDA;
    mpq_context* c = new (std::nothrow) mpq_context();
    if (!c) return MPQ_ERR_CUDA;
    c->magic = CTX_MAGIC;
    c->device = device;
    c->launches = 0;
    c->hx = c->hy = nullptr;
    c->hx_bytes = c->hy_bytes = 0;
    c->q4_partials = nullptr;
    c->q4_partials_warps = 0;
    c->q4_status = nullptr;
    if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&c->prop, device) != cudaSuccess) {
        delete c;
        return MPQ_ERR_CUDA;
    }
    if (c->prop.major != 10) {   // sm_100a code only; no other path exists
        delete c;
        return MPQ_ERR_UNSUPPORTED;
    }
    const char* e = getenv("MPQ_PDL");
    c->pdl = !(e && e[0] == '0');
    e = getenv("MPQ_Q4_VARIANT");
    c->q4_variant = (e && e[0] == '1') ? 1 : 0;
    e = getenv("MPQ_Q4_STREAM");
    c->q4_stream = !(e && e[0] == '0');
    e = getenv("MPQ_Q4_GROUP");
    c->q4_group = (e && e[0] == '4') ? 4 : 2;
    e = getenv("MPQ_Q4_DEPTH");
    c->q4_depth = (e && e[0] >= '1' && e[0] <= '4') ? e[0] - '0' : 2;
    e = getenv("MPQ_Q4_PRE");
    c->q4_pre = (e && e[0] >= '0' && e[0] <= '4') ? e[0] - '0' : 1;
    e = getenv("MPQ_Q4_SLAB4");
    c->q4_slab4 = !(e && e[0] == '0');
    e = getenv("MPQ_Q4_TILE");
    c->q4_tile_mode = !(e && e[0] == '0');
    *out = c;
    return MPQ_OK;
}

extern "C" int32_t mpq_context_destroy(mpq_context* ctx)
{
    if (!ctx_ok(ctx)) return MPQ_ERR_INVALID_ARG;
    cudaSetDevice(ctx->device);
    cudaFree(ctx->hx);
    cudaFree(ctx->hy);
    cudaFree(ctx->q4_partials);
    cudaFree(ctx->q4_status);
    ctx->fp4.release();
    ctx->magic = 0;
    delete ctx;
    return MPQ_OK;
}

extern "C" int32_t mpq_context_info(const mpq_context* ctx, mpq_device_info* out)
{
    if (!ctx_ok(ctx) || !out) return MPQ_ERR_INVALID_ARG;
    out->device = ctx->device;
    out->sm_count = ctx->prop.multiProcessorCount;
    out->cc_major = ctx->prop.major;
    out->cc_minor = ctx->prop.minor;
    out->l2_bytes = ctx->prop.l2CacheSize;
    out->total_mem_bytes = (int64_t)ctx->prop.totalGlobalMem;
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, ctx->device);
    out->sm_clock_khz = v;
    cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, ctx->device);
    out->mem_clock_khz = v;
    return MPQ_OK;
}

extern "C" const char* mpq_last_error(const mpq_context* ctx) { return ctx_ok(ctx) ? ctx->err.c_str() : "invalid context"; }
extern "C" int64_t mpq_context_launch_count(const mpq_context* ctx) { return ctx_ok(ctx) ? ctx->launches : -1; }

// ---------------------------------------------------------------------------
// Q4 weights
// ---------------------------------------------------------------------------
static int32_t q4_build(mpq_context* ctx, int64_t Nfull, int64_t Kfull, const uint8_t* codes_dev, const uint16_t* scales_dev,
                        int64_t row0, int64_t k0, int64_t N, int64_t K, mpq_weight** out)
{
    mpq_weight* w = new (std::nothrow) mpq_weight();
    if (!w) return fail(ctx, MPQ_ERR_CUDA, "out of host memory");
    (void)Nfull;
    w->magic = W_MAGIC;
    w->fmt = MPQ_FMT_Q4;
    w->device = ctx->device;
    Q4Dev& q = w->q4;
    q.N = N;
    q.K = K;
    q.nrp = (int)((N + 31) / 32);
    q.nchunks = (int)((K + 63) / 64);
    q.nchunks = (q.nchunks + Q4_GROUP_PAD - 1) / Q4_GROUP_PAD * Q4_GROUP_PAD;   // a bulk-copy group never straddles a row pair-tile
    cudaError_t e = cudaMalloc(&q.stream, q.bytes());
    if (e != cudaSuccess) {
        delete w;
        return fail(ctx, MPQ_ERR_CUDA, "cudaMalloc of %zu weight bytes failed: %s", q.bytes(), cudaGetErrorString(e));
    }
    int64_t words = (int64_t)q.nrp * q.nchunks * 256, halves = (int64_t)q.nrp * q.nchunks * 64;
    q4_repack_codes_kernel<<<(unsigned)((words + 255) / 256), 256>>>(codes_dev, Kfull, row0, k0, N, K, q.nrp, q.nchunks,
                                                                      reinterpret_cast<uint32_t*>(q.stream));
    q4_repack_scales_kernel<<<(unsigned)((halves + 255) / 256), 256>>>(scales_dev, Kfull / 32, row0, k0 / 32, N, K / 32, q.nrp,
                                                                        q.nchunks, reinterpret_cast<uint16_t*>(q.stream));
    ctx->launches += 2;
    e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(q.stream);
        delete w;
        return fail(ctx, MPQ_ERR_CUDA, "Q4 repack failed: %s", cudaGetErrorString(e));
    }
    *out = w;
    return MPQ_OK;
}

static int32_t q4_shard(mpq_context* ctx, int64_t N, int64_t K, int32_t tp_mode, int32_t rank, int32_t world,
                        int64_t* row0, int64_t* k0, int64_t* n, int64_t* k)
{
    *row0 = 0; *k0 = 0; *n = N; *k = K;
    if (world < 1 || rank < 0 || rank >= world) return fail(ctx, MPQ_ERR_INVALID_ARG, "rank %d / world %d", rank, world);
    if (tp_mode == MPQ_TP_NONE) {
        if (world != 1) return fail(ctx, MPQ_ERR_INVALID_ARG, "tp_mode NONE needs world == 1");
    } else if (tp_mode == MPQ_TP_COLUMN) {
        if (N % world) return fail(ctx, MPQ_ERR_SHAPE, "N=%lld not divisible by world=%d", (long long)N, world);
        *n = N / world; *row0 = *n * rank;
    } else if (tp_mode == MPQ_TP_ROW) {
        if (K % (32LL * world)) return fail(ctx, MPQ_ERR_SHAPE, "K=%lld: K/world must be a multiple of 32", (long long)K);
        *k = K / world; *k0 = *k * rank;
    } else
        return fail(ctx, MPQ_ERR_INVALID_ARG, "tp_mode %d", tp_mode);
    return MPQ_OK;
}

extern "C" int32_t mpq_q4_weight_create(mpq_context* ctx, int64_t N, int64_t K, const uint8_t* codes_host,
                                        const uint16_t* scales_host, int32_t tp_mode, int32_t rank, int32_t world,
                                        mpq_weight** out)
{
    if (!ctx_ok(ctx)) return MPQ_ERR_INVALID_ARG;
    if (!out || !codes_host || !scales_host) return fail(ctx, MPQ_ERR_INVALID_ARG, "null pointer");
    *out = nullptr;
    if (N <= 0 || K <= 0 || K % 32) return fail(ctx, MPQ_ERR_SHAPE, "Q4 needs N > 0 and K a positive multiple of 32 (N=%lld K=%lld)", (long long)N, (long long)K);
    if (N > (1LL << 30) || K > (1LL << 30)) return fail(ctx, MPQ_ERR_UNSUPPORTED, "dimension above 2^30");
    int64_t row0, k0, n, k;
    int32_t st = q4_shard(ctx, N, K, tp_mode, rank, world, &row0, &k0, &n, &k);
    if (st) return st;
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    // upload only the rows the shard needs (all K of them; the K slice is cut by the repack)
    size_t cb = (size_t)n * (K / 2), sb = (size_t)n * (K / 32) * 2;
    uint8_t* dc = nullptr;
    uint16_t* ds = nullptr;
    CU_TRY(ctx, cudaMalloc(&dc, cb));
    cudaError_t e = cudaMalloc(&ds, sb);
    if (e == cudaSuccess) e = cudaMemcpy(dc, codes_host + (size_t)row0 * (K / 2), cb, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(ds, scales_host + (size_t)row0 * (K / 32), sb, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaFree(dc);
        cudaFree(ds);
        return fail(ctx, MPQ_ERR_CUDA, "upload of canonical Q4 arrays failed: %s", cudaGetErrorString(e));
    }
    st = q4_build(ctx, n, K, dc, ds, 0, k0, n, k, out);
    cudaFree(dc);
    cudaFree(ds);
    return st;
}

extern "C" int32_t mpq_q4_weight_create_dev(mpq_context* ctx, int64_t N, int64_t K, const uint8_t* codes_dev,
                                            const uint16_t* scales_dev, mpq_weight** out)
{
    if (!ctx_ok(ctx)) return MPQ_ERR_INVALID_ARG;
    if (!out || !codes_dev || !scales_dev) return fail(ctx, MPQ_ERR_INVALID_ARG, "null pointer");
    *out = nullptr;
    if (N <= 0 || K <= 0 || K % 32) return fail(ctx, MPQ_ERR_SHAPE, "Q4 needs N > 0 and K a positive multiple of 32 (N=%lld K=%lld)", (long long)N, (long long)K);
    if (N > (1LL << 30) || K > (1LL << 30)) return fail(ctx, MPQ_ERR_UNSUPPORTED, "dimension above 2^30");
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    return q4_build(ctx, N, K, codes_dev, scales_dev, 0, 0, N, K, out);
}

// ---------------------------------------------------------------------------
// any weight
// ---------------------------------------------------------------------------
extern "C" int32_t mpq_weight_shape(const mpq_weight* w, int64_t* N, int64_t* K, int32_t* fmt)
{
    if (!w_ok(w)) return MPQ_ERR_INVALID_ARG;
    if (N) *N = w->fmt == MPQ_FMT_Q4 ? w->q4.N : w->fp4.N;
    if (K) *K = w->fmt == MPQ_FMT_Q4 ? w->q4.K : w->fp4.K;
    if (fmt) *fmt = w->fmt;
    return MPQ_OK;
}

extern "C" int64_t mpq_weight_device_bytes(const mpq_weight* w)
{
    if (!w_ok(w)) return -1;
    return w->fmt == MPQ_FMT_Q4 ? (int64_t)w->q4.bytes() : (int64_t)w->fp4.device_bytes();
}

extern "C" int32_t mpq_weight_destroy(mpq_weight* w)
{
    if (!w_ok(w)) return MPQ_ERR_INVALID_ARG;
    cudaSetDevice(w->device);
    cudaFree(w->q4.stream);
    w->fp4.release();
    w->magic = 0;
    delete w;
    return MPQ_OK;
}

extern "C" int32_t mpq_weight_dequantize(mpq_context* ctx, const mpq_weight* w, float* out_dev, void* stream)
{
    if (!ctx_ok(ctx)) return MPQ_ERR_INVALID_ARG;
    if (!w_ok(w) || !out_dev) return fail(ctx, MPQ_ERR_INVALID_ARG, "null or stale handle");
    if (w->device != ctx->device) return fail(ctx, MPQ_ERR_INVALID_ARG, "weight lives on device %d, context on %d", w->device, ctx->device);
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    cudaStream_t s = (cudaStream_t)stream;
    if (w->fmt == MPQ_FMT_Q4) {
        const Q4Dev& q = w->q4;
        int64_t words = (int64_t)q.nrp * q.nchunks * 256;
        q4_dequant_kernel<<<(unsigned)((words + 255) / 256), 256, 0, s>>>(reinterpret_cast<const uint32_t*>(q.stream), q.N, q.K,
                                                                           q.nrp, q.nchunks, out_dev);
    } else {
        const Nvfp4Dev& f = w->fp4;
        nvfp4_dequant_launch(f.codes, f.sf_canonical, f.tensor_scale, f.N, f.K, out_dev, s);
    }
    ctx->launches += 1;
    CU_TRY(ctx, cudaGetLastError());
    return MPQ_OK;
}

// ---------------------------------------------------------------------------
// Q4 linear
// ---------------------------------------------------------------------------
template <int MT, bool SUBN>
static cudaError_t q4_launch_t(const Q4Launch& p, dim3 grid, size_t smem, bool pdl, cudaStream_t s)
{
    auto kern = q4_linear_kernel<MT, SUBN>;
    static bool configured = false;        // per instantiation; static + dynamic shared memory may pass 48 KiB
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(160 * 1024));
        if (e != cudaSuccess) return e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(Q4_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[2];
    int na = 0;
    if (p.splits > 1) {
        at[na].id = cudaLaunchAttributeClusterDimension;
        at[na].val.clusterDim.x = 1;
        at[na].val.clusterDim.y = (unsigned)p.splits;
        at[na].val.clusterDim.z = 1;
        ++na;
    }
    if (pdl) {
        at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = at;
    cfg.numAttrs = (unsigned)na;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

// Scratch of the streaming kernel, allocated on first use and kept for the context's life.
static const int Q4S_MAX_WARPS = 32 * 1024;    // up to four CTAs of 8 warps on up to 1024 SMs
static int32_t q4_stream_scratch(mpq_context* ctx, int warps)
{
    if (!ctx->q4_status) {
        CU_TRY(ctx, cudaMalloc(&ctx->q4_status, sizeof(int)));
        CU_TRY(ctx, cudaMemset(ctx->q4_status, 0, sizeof(int)));
    }
    if (ctx->q4_partials_warps < warps) {
        CU_TRY(ctx, cudaDeviceSynchronize());          // nobody may still be using the old array
        cudaFree(ctx->q4_partials);
        ctx->q4_partials = nullptr;
        ctx->q4_partials_warps = 0;
        int n = std::max(warps, 4096);
        size_t bytes = (size_t)n * 2 * 32 * 4 * sizeof(uint2);
        CU_TRY(ctx, cudaMalloc(&ctx->q4_partials, bytes));
        CU_TRY(ctx, cudaMemset(ctx->q4_partials, 0, bytes));      // tag 0 = empty slot
        ctx->q4_partials_warps = n;
    }
    return MPQ_OK;
}

// The streaming kernel applies when M <= 4 and the staged activation plus a ring fit in shared memory.
struct Q4StreamPlan { int depth, G, nx, ctas_per_sm; size_t smem; };
static bool q4_stream_plan(const mpq_context* ctx, const Q4Dev& q, int M, Q4StreamPlan* pl)
{
    if (!ctx->q4_stream || M > 4) return false;
    size_t nblk = (size_t)q.nchunks * 2;
    size_t xbytes = nblk * (2 * M) * 64 + nblk * M * 16 + 8 * 8 * Q4S_WARPS;
    int need = (M * q.nchunks + 31) / 32;                 // float4 of x per thread (512 threads)
    pl->nx = need <= 4 ? 4 : need <= 8 ? 8 : need <= 16 ? 16 : 0;
    pl->ctas_per_sm = 1;
    // one CTA per SM: 227 KiB less the kernel's static shared memory (17 KiB) and the 1 KiB the system reserves
    const size_t budget = (size_t)(227 - 18) * 1024;
    const int prefer = ctx->q4_group;
    for (int pass = 0; pass < 2; ++pass) {
        const int G = pass == 0 ? prefer : (prefer == 4 ? 2 : 4);
        const size_t stage = (size_t)Q4S_WARPS * G * Q4_UNIT_BYTES;
        for (int d = std::min(ctx->q4_depth, G == 4 ? 2 : 4); d >= 1; --d) {
            size_t total = stage * d + xbytes;
            if (total <= budget) { pl->G = G; pl->depth = d; pl->smem = total; return true; }
        }
    }
    return false;
}

template <bool SUBN, int G, int NX, int MINB>
static cudaError_t q4_stream_launch_t(const Q4StreamLaunch& p, int grid, size_t smem, bool pdl, cudaStream_t s)
{
    auto kern = q4_stream_kernel<SUBN, G, NX, MINB>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(209 * 1024));
        if (e != cudaSuccess) return e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(Q4S_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1u : 0u;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

template <bool SUBN, int G>
static cudaError_t q4_stream_launch_nx(int nx, const Q4StreamLaunch& p, int grid, size_t smem, bool pdl, cudaStream_t s)
{
    switch (nx) {
        case 4: return q4_stream_launch_t<SUBN, G, 4, 1>(p, grid, smem, pdl, s);
        case 8: return q4_stream_launch_t<SUBN, G, 8, 1>(p, grid, smem, pdl, s);
        case 16: return q4_stream_launch_t<SUBN, G, 16, 1>(p, grid, smem, pdl, s);
        default: return q4_stream_launch_t<SUBN, G, 0, 1>(p, grid, smem, pdl, s);
    }
}

// The streaming kernel for one slab of M <= 4 rows; with an exchange it also adds the ranks' partial outputs.
static int32_t q4_stream_forward(mpq_context* ctx, const Q4Dev& q, const Q4StreamPlan& pl, const float* x, int M, float* y,
                                 int64_t ldy, mpq_exchange* ex, cudaStream_t s)
{
    {
        const int sms = ctx->prop.multiProcessorCount;
        const int groups = (int)(q.units() / pl.G);
        int W = (int)std::min<int64_t>((int64_t)sms * Q4S_WARPS, groups);
        W = std::min(W, Q4S_MAX_WARPS);
        int32_t st = q4_stream_scratch(ctx, W);
        if (st) return st;
        Q4StreamLaunch p;
        // whole row pair-tiles per CTA when there is about one per SM or more: no tile is then shared between CTAs
        p.tile_mode = (ctx->q4_tile_mode && (int64_t)q.nrp * 10 >= (int64_t)sms * 6) ? 1 : 0;
        p.nrp = q.nrp;
        p.stream = q.stream; p.X = x; p.Y = y; p.M = M; p.N = (int)q.N; p.K = (int)q.K; p.ldy = ldy;
        p.nchunks = q.nchunks; p.groups = groups; p.warps_total = W; p.depth = pl.depth; p.pre = ctx->q4_pre;
        p.partials = ctx->q4_partials; p.status = ctx->q4_status;
        p.xworld = 0; p.xrank = 0; p.xslot = 0; p.xlimit = 0;
        for (int r = 0; r < 8; ++r) p.xpeer[r] = nullptr;
        if (ex) {
            const size_t half = (size_t)(++ex->calls & 1u) * ex->world * ex->max_floats;
            p.xworld = ex->world; p.xrank = ex->rank; p.xslot = ex->max_floats; p.xlimit = ex->wait_limit;
            for (int r = 0; r < ex->world; ++r) p.xpeer[r] = ex->peer[r] + half;
        }
        int grid = p.tile_mode ? std::min(sms, q.nrp) : (W + Q4S_WARPS - 1) / Q4S_WARPS;
        cudaError_t e;
        const bool subn = ctx->q4_variant == 0;
        if (pl.G == 4) e = subn ? q4_stream_launch_nx<true, 4>(pl.nx, p, grid, pl.smem, ctx->pdl, s) : q4_stream_launch_nx<false, 4>(pl.nx, p, grid, pl.smem, ctx->pdl, s);
        else e = subn ? q4_stream_launch_nx<true, 2>(pl.nx, p, grid, pl.smem, ctx->pdl, s) : q4_stream_launch_nx<false, 2>(pl.nx, p, grid, pl.smem, ctx->pdl, s);
        ctx->launches += 1;
        if (e != cudaSuccess) return fail(ctx, MPQ_ERR_CUDA, "q4_stream_kernel launch failed: %s", cudaGetErrorString(e));
        return MPQ_OK;
    }
}

// One launch for a slab of M <= 16 activation rows.
static int32_t q4_forward_general(mpq_context* ctx, const Q4Dev& q, const float* x, int M, float* y, int64_t ldy, cudaStream_t s);
static int32_t q4_forward_slab(mpq_context* ctx, const Q4Dev& q, const float* x, int M, float* y, int64_t ldy, cudaStream_t s)
{
    Q4StreamPlan pl;
    if (q4_stream_plan(ctx, q, M, &pl)) return q4_stream_forward(ctx, q, pl, x, M, y, ldy, nullptr, s);
    return q4_forward_general(ctx, q, x, M, y, ldy, s);
}

// The phase-staged kernel: any M <= 16, any K; needs no scratch memory.
static int32_t q4_forward_general(mpq_context* ctx, const Q4Dev& q, const float* x, int M, float* y, int64_t ldy, cudaStream_t s)
{
    const int MT = M <= 4 ? 1 : (M <= 8 ? 2 : 4);
    const int sms = ctx->prop.multiProcessorCount;
    // K split across a thread-block cluster until the grid covers the machine about three times
    int splits = 1;
    while (splits < 8 && (int64_t)q.nrp * splits < 3LL * sms && q.nchunks / (splits * 2) >= Q4_WARPS) splits *= 2;
    int cpc = (q.nchunks + splits - 1) / splits;
    const size_t per_chunk = (size_t)2 * (2 * M) * 64 + (size_t)2 * MT * 64;   // xs + cs bytes per chunk
    const size_t cap = M <= 4 ? 64 * 1024 : 96 * 1024;
    int cpp = (int)std::min<size_t>((size_t)cpc, std::max<size_t>(Q4_WARPS, cap / per_chunk));
    size_t smem = per_chunk * cpp;

    Q4Launch p;
    p.stream = q.stream; p.X = x; p.Y = y;
    p.M = M; p.N = (int)q.N; p.K = (int)q.K; p.ldy = ldy;
    p.nchunks = q.nchunks; p.chunks_per_cta = cpc; p.chunks_per_phase = cpp; p.splits = splits;
    dim3 grid((unsigned)q.nrp, (unsigned)splits);
    cudaError_t e;
    const bool subn = ctx->q4_variant == 0;
    if (MT == 1) e = subn ? q4_launch_t<1, true>(p, grid, smem, ctx->pdl, s) : q4_launch_t<1, false>(p, grid, smem, ctx->pdl, s);
    else if (MT == 2) e = subn ? q4_launch_t<2, true>(p, grid, smem, ctx->pdl, s) : q4_launch_t<2, false>(p, grid, smem, ctx->pdl, s);
    else e = subn ? q4_launch_t<4, true>(p, grid, smem, ctx->pdl, s) : q4_launch_t<4, false>(p, grid, smem, ctx->pdl, s);
    ctx->launches += 1;
    if (e != cudaSuccess) return fail(ctx, MPQ_ERR_CUDA, "q4_linear_kernel launch failed: %s", cudaGetErrorString(e));
    return MPQ_OK;
}

// Rows per launch for M activation rows: the streaming kernel's widest slab (4, 2 or 1 rows) whose staged
// activation fits in shared memory, else 16 through the phase-staged kernel.
static int q4_slab_rows(const mpq_context* ctx, const Q4Dev& q, int64_t M)
{
    Q4StreamPlan pl;
    if (M <= 4 && q4_stream_plan(ctx, q, (int)M, &pl)) return (int)M;      // one launch of the streaming kernel
    if (ctx->q4_slab4 && M > 1) {
        const int widths[3] = {4, 2, 1};
        for (int i = 0; i < 3; ++i)
            if (widths[i] < M && q4_stream_plan(ctx, q, widths[i], &pl)) return widths[i];
    }
    return 16;
}

static int32_t q4_forward_checked(mpq_context* ctx, const mpq_weight* w, const float* x_dev, int64_t M, float* y_dev,
                                  int64_t ldy, cudaStream_t s)
{
    // M > 4: slabs of four rows through the streaming kernel where it applies (it re-reads the weights per
    // slab but runs near the HBM roofline), else slabs of sixteen through the phase-staged kernel, whose
    // legacy-MMA arithmetic is the bound from M = 8 up.
    const int slab = q4_slab_rows(ctx, w->q4, M);
    for (int64_t m0 = 0; m0 < M; m0 += slab) {
        int m = (int)std::min<int64_t>(slab, M - m0);
        int32_t st = q4_forward_slab(ctx, w->q4, x_dev + (size_t)m0 * w->q4.K, m, y_dev + (size_t)m0 * ldy, ldy, s);
        if (st) return st;
    }
    return MPQ_OK;
}

static int32_t q4_validate(mpq_context* ctx, const mpq_weight* w, const void* x, int64_t M, const void* y)
{
    if (!ctx_ok(ctx)) return MPQ_ERR_INVALID_ARG;
    if (!w_ok(w) || !x || !y) return fail(ctx, MPQ_ERR_INVALID_ARG, "null or stale handle / pointer");
    if (w->fmt != MPQ_FMT_Q4) return fail(ctx, MPQ_ERR_INVALID_ARG, "weight is not Q4");
    if (w->device != ctx->device) return fail(ctx, MPQ_ERR_INVALID_ARG, "weight lives on device %d, context on %d", w->device, ctx->device);
    if (M <= 0 || M > (1 << 20)) return fail(ctx, MPQ_ERR_SHAPE, "M=%lld out of range", (long long)M);
    return MPQ_OK;
}

extern "C" int32_t mpq_q4_linear_forward(mpq_context* ctx, const mpq_weight* w, const float* x_dev, int64_t M,
                                         float* y_dev, void* stream)
{
    int32_t st = q4_validate(ctx, w, x_dev, M, y_dev);
    if (st) return st;
    if (!aligned16(x_dev) || !aligned16(y_dev)) return fail(ctx, MPQ_ERR_ALIGN, "x and y must be 16-byte aligned");
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    return q4_forward_checked(ctx, w, x_dev, M, y_dev, w->q4.N, (cudaStream_t)stream);
}

static int32_t grow(mpq_context* ctx, float** buf, size_t* have, size_t need)
{
    if (*have >= need) return MPQ_OK;
    cudaFree(*buf);
    *buf = nullptr;
    *have = 0;
    CU_TRY(ctx, cudaMalloc(buf, need));
    *have = need;
    return MPQ_OK;
}

extern "C" int32_t mpq_q4_linear_forward_host(mpq_context* ctx, const mpq_weight* w, const float* x_host, int64_t M,
                                              float* y_host)
{
    int32_t st = q4_validate(ctx, w, x_host, M, y_host);
    if (st) return st;
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    size_t xb = (size_t)M * w->q4.K * 4, yb = (size_t)M * w->q4.N * 4;
    if ((st = grow(ctx, &ctx->hx, &ctx->hx_bytes, xb))) return st;
    if ((st = grow(ctx, &ctx->hy, &ctx->hy_bytes, yb))) return st;
    CU_TRY(ctx, cudaMemcpyAsync(ctx->hx, x_host, xb, cudaMemcpyHostToDevice, 0));
    if ((st = q4_forward_checked(ctx, w, ctx->hx, M, ctx->hy, w->q4.N, 0))) return st;
    CU_TRY(ctx, cudaMemcpyAsync(y_host, ctx->hy, yb, cudaMemcpyDeviceToHost, 0));
    CU_TRY(ctx, cudaStreamSynchronize(0));
    return MPQ_OK;
}

// ---------------------------------------------------------------------------
// Q4 linear without any allocation
// ---------------------------------------------------------------------------
// Some callers cannot let the library allocate: a host thread that replays work inside a fixed memory
// budget, a real-time loop that must not enter the allocator's locks, code that runs while another
// thread holds the device in a state where cudaMalloc would synchronise.  mpq_q4_linear_forward
// allocates lazily (the streaming kernel's scratch, on a context's first call); this variant never
// does.  Its scratch is the array below, which every GPU that loads the library holds until exit.
constexpr int Q4_STATIC_MAX_CTAS = 512;                                   // two CTAs per SM on up to 256 SMs
constexpr size_t Q4_STATIC_SLOT_BYTES = (size_t)Q4_STATIC_MAX_CTAS * 2 * 32 * 4 * sizeof(uint2);   // 1 MiB
static __device__ __align__(256) unsigned char g_q4_static_scratch[256 + Q4_STATIC_SLOT_BYTES];
// In host code the array's name is only a stand-in: the device address comes from cudaGetSymbolAddress,
// once per device, with that device current.
static unsigned char* g_q4_static_ptr[64] = {};

extern "C" int32_t mpq_q4_linear_forward_static(mpq_context* ctx, const mpq_weight* w, const float* x_dev, int64_t M,
                                                float* y_dev, int32_t* status_dev, void* stream)
{
    int32_t st = q4_validate(ctx, w, x_dev, M, y_dev);
    if (st) return st;
    if (!aligned16(x_dev) || !aligned16(y_dev)) return fail(ctx, MPQ_ERR_ALIGN, "x and y must be 16-byte aligned");
    if (ctx->device < 0 || ctx->device >= 64) return fail(ctx, MPQ_ERR_UNSUPPORTED, "device index %d beyond the static table", ctx->device);
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    if (!g_q4_static_ptr[ctx->device]) {                  // set-up: the first call on this device
        void* p = nullptr;
        CU_TRY(ctx, cudaGetSymbolAddress(&p, g_q4_static_scratch));
        g_q4_static_ptr[ctx->device] = static_cast<unsigned char*>(p);
    }
    unsigned char* base = g_q4_static_ptr[ctx->device];
    const Q4Dev& q = w->q4;
    cudaStream_t s = (cudaStream_t)stream;
    const int slab = q4_slab_rows(ctx, q, M);          // the same split into launches as mpq_q4_linear_forward
    for (int64_t m0 = 0; m0 < M; m0 += slab) {
        const int m = (int)std::min<int64_t>(slab, M - m0);
        const float* x = x_dev + (size_t)m0 * q.K;
        float* y = y_dev + (size_t)m0 * q.N;
        Q4StreamPlan pl;
        if (!q4_stream_plan(ctx, q, m, &pl)) {            // the phase-staged kernel uses no scratch at all
            st = q4_forward_general(ctx, q, x, m, y, q.N, s);
            if (st) return st;
            continue;
        }
        const int sms = ctx->prop.multiProcessorCount;
        const int groups = (int)(q.units() / pl.G);
        const int W = (int)std::min<int64_t>((int64_t)sms * Q4S_WARPS, groups);
        const int tile_mode = (ctx->q4_tile_mode && (int64_t)q.nrp * 10 >= (int64_t)sms * 6) ? 1 : 0;
        const int grid = tile_mode ? std::min(sms, q.nrp) : (W + Q4S_WARPS - 1) / Q4S_WARPS;
        if (grid > Q4_STATIC_MAX_CTAS)
            return fail(ctx, MPQ_ERR_UNSUPPORTED, "this launch needs %d scratch slots, the static array holds %d", grid, Q4_STATIC_MAX_CTAS);
        Q4StreamLaunch p;
        p.stream = q.stream; p.X = x; p.Y = y; p.M = m; p.N = (int)q.N; p.K = (int)q.K; p.ldy = q.N;
        p.nchunks = q.nchunks; p.groups = groups; p.warps_total = W; p.depth = pl.depth; p.pre = ctx->q4_pre;
        p.tile_mode = tile_mode; p.nrp = q.nrp;
        p.partials = reinterpret_cast<uint2*>(base + 256);
        p.status = status_dev ? status_dev : reinterpret_cast<int*>(base);
        p.xworld = 0; p.xrank = 0; p.xslot = 0; p.xlimit = 0;
        for (int r = 0; r < 8; ++r) p.xpeer[r] = nullptr;
        cudaError_t e;
        const bool subn = ctx->q4_variant == 0;
        if (pl.G == 4) e = subn ? q4_stream_launch_nx<true, 4>(pl.nx, p, grid, pl.smem, ctx->pdl, s) : q4_stream_launch_nx<false, 4>(pl.nx, p, grid, pl.smem, ctx->pdl, s);
        else e = subn ? q4_stream_launch_nx<true, 2>(pl.nx, p, grid, pl.smem, ctx->pdl, s) : q4_stream_launch_nx<false, 2>(pl.nx, p, grid, pl.smem, ctx->pdl, s);
        ctx->launches += 1;
        if (e != cudaSuccess) return fail(ctx, MPQ_ERR_CUDA, "q4_stream_kernel launch failed: %s", cudaGetErrorString(e));
    }
    return MPQ_OK;
}

// ---------------------------------------------------------------------------
// tensor-parallel exchange
// ---------------------------------------------------------------------------
extern "C" int32_t mpq_exchange_create(mpq_context* ctx, int32_t rank, int32_t world, int64_t max_floats, mpq_exchange** out)
{
    if (!ctx_ok(ctx)) return MPQ_ERR_INVALID_ARG;
    if (!out) return fail(ctx, MPQ_ERR_INVALID_ARG, "null pointer");
    *out = nullptr;
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(ctx, MPQ_ERR_INVALID_ARG, "rank %d / world %d (world <= 8)", rank, world);
    if (max_floats <= 0 || max_floats > (1LL << 26)) return fail(ctx, MPQ_ERR_SHAPE, "max_floats=%lld out of range", (long long)max_floats);
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    mpq_exchange* x = new (std::nothrow) mpq_exchange();
    if (!x) return fail(ctx, MPQ_ERR_CUDA, "out of host memory");
    x->magic = X_MAGIC; x->device = ctx->device; x->rank = rank; x->world = world; x->max_floats = max_floats;
    x->calls = 0; x->wait_limit = 1u << 22; x->attached = world == 1;
    for (int r = 0; r < 8; ++r) { x->peer[r] = nullptr; x->opened[r] = false; }
    size_t bytes = (size_t)2 * world * max_floats * sizeof(uint2);
    cudaError_t e = cudaMalloc(&x->local, bytes);
    if (e == cudaSuccess) e = cudaMemset(x->local, 0, bytes);          // tag 0 = empty slot
    if (e != cudaSuccess) {
        cudaFree(x->local);
        delete x;
        return fail(ctx, MPQ_ERR_CUDA, "exchange allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    }
    x->peer[rank] = x->local;
    *out = x;
    return MPQ_OK;
}

extern "C" int32_t mpq_exchange_ipc_handle(mpq_exchange* x, uint8_t* out64)
{
    if (!x_ok(x) || !out64) return MPQ_ERR_INVALID_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    if (cudaSetDevice(x->device) != cudaSuccess || cudaIpcGetMemHandle(&h, x->local) != cudaSuccess) return MPQ_ERR_CUDA;
    memcpy(out64, &h, 64);
    return MPQ_OK;
}

extern "C" int32_t mpq_exchange_attach(mpq_exchange* x, const uint8_t* handles)
{
    if (!x_ok(x) || !handles) return MPQ_ERR_INVALID_ARG;
    if (x->attached) return MPQ_ERR_STATE;
    if (cudaSetDevice(x->device) != cudaSuccess) return MPQ_ERR_CUDA;
    for (int r = 0; r < x->world; ++r) {
        if (r == x->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + 64 * r, 64);
        void* p = nullptr;
        if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return MPQ_ERR_CUDA; }
        x->peer[r] = reinterpret_cast<uint2*>(p);
        x->opened[r] = true;
    }
    x->attached = true;
    return MPQ_OK;
}

extern "C" int32_t mpq_exchange_attach_pointers(mpq_exchange* x, void* const* buffers)
{
    if (!x_ok(x) || !buffers) return MPQ_ERR_INVALID_ARG;
    if (x->attached) return MPQ_ERR_STATE;
    for (int r = 0; r < x->world; ++r) {
        if (r == x->rank) continue;
        if (!buffers[r]) return MPQ_ERR_INVALID_ARG;
        x->peer[r] = reinterpret_cast<uint2*>(buffers[r]);
    }
    x->attached = true;
    return MPQ_OK;
}

extern "C" int32_t mpq_exchange_buffer(mpq_exchange* x, void** dev_ptr, int64_t* bytes)
{
    if (!x_ok(x)) return MPQ_ERR_INVALID_ARG;
    if (dev_ptr) *dev_ptr = x->local;
    if (bytes) *bytes = (int64_t)2 * x->world * x->max_floats * (int64_t)sizeof(uint2);
    return MPQ_OK;
}

extern "C" int32_t mpq_exchange_set_wait_limit(mpq_exchange* x, uint32_t polls)
{
    if (!x_ok(x) || polls == 0) return MPQ_ERR_INVALID_ARG;
    x->wait_limit = polls;
    return MPQ_OK;
}

extern "C" int32_t mpq_exchange_destroy(mpq_exchange* x)
{
    if (!x_ok(x)) return MPQ_ERR_INVALID_ARG;
    cudaSetDevice(x->device);
    for (int r = 0; r < x->world; ++r)
        if (x->opened[r]) cudaIpcCloseMemHandle(x->peer[r]);
    cudaFree(x->local);
    x->magic = 0;
    delete x;
    return MPQ_OK;
}

extern "C" int32_t mpq_q4_linear_forward_allreduce(mpq_context* ctx, const mpq_weight* w, mpq_exchange* ex, const float* x_dev,
                                                   int64_t M, float* y_dev, void* stream)
{
    int32_t st = q4_validate(ctx, w, x_dev, M, y_dev);
    if (st) return st;
    if (!x_ok(ex)) return fail(ctx, MPQ_ERR_INVALID_ARG, "null or stale exchange");
    if (ex->device != ctx->device) return fail(ctx, MPQ_ERR_INVALID_ARG, "exchange lives on device %d, context on %d", ex->device, ctx->device);
    if (!ex->attached) return fail(ctx, MPQ_ERR_STATE, "exchange used before its peers were attached");
    if (!aligned16(x_dev) || !aligned16(y_dev)) return fail(ctx, MPQ_ERR_ALIGN, "x and y must be 16-byte aligned");
    if (M * w->q4.N > ex->max_floats) return fail(ctx, MPQ_ERR_UNSUPPORTED, "M*N=%lld exceeds the exchange capacity %lld", (long long)(M * w->q4.N), (long long)ex->max_floats);
    Q4StreamPlan pl;
    if (M > 4 || !q4_stream_plan(ctx, w->q4, (int)M, &pl))
        return fail(ctx, MPQ_ERR_UNSUPPORTED, "the fused all-reduce needs M <= 4 and an activation that fits in shared memory");
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    return q4_stream_forward(ctx, w->q4, pl, x_dev, (int)M, y_dev, w->q4.N, ex, (cudaStream_t)stream);
}

extern "C" int32_t mpq_context_poll_status(mpq_context* ctx)
{
    if (!ctx_ok(ctx)) return MPQ_ERR_INVALID_ARG;
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    int* words[2] = {ctx->q4_status, ctx->fp4.status};
    for (int i = 0; i < 2; ++i) {
        if (!words[i]) continue;
        int v = 0;
        CU_TRY(ctx, cudaMemcpy(&v, words[i], sizeof(int), cudaMemcpyDeviceToHost));    // synchronises with prior work
        if (v == 0) continue;
        cudaMemset(words[i], 0, sizeof(int));            // a wait ran out: clear the word for the next launch
        if (i == 0 && ctx->q4_partials)                  // ... and the slots the aborted launch may have left full
            cudaMemset(ctx->q4_partials, 0, (size_t)ctx->q4_partials_warps * 2 * 32 * 4 * sizeof(uint2));
        return fail(ctx, MPQ_ERR_PEER_TIMEOUT, "a bounded device-side wait ran out (%s kernel, code %d)", i ? "NVFP4 GEMM" : "Q4", v);
    }
    return MPQ_OK;
}

// ---------------------------------------------------------------------------
// NVFP4
// ---------------------------------------------------------------------------
extern "C" int32_t mpq_nvfp4_weight_create(mpq_context* ctx, int64_t N, int64_t K, const uint8_t* codes_host,
                                           const uint8_t* sf_host, float tensor_scale, mpq_weight** out)
{
    if (!ctx_ok(ctx)) return MPQ_ERR_INVALID_ARG;
    if (!out || !codes_host || !sf_host) return fail(ctx, MPQ_ERR_INVALID_ARG, "null pointer");
    *out = nullptr;
    if (N <= 0 || K <= 0 || N % 8 || K % 32)
        return fail(ctx, MPQ_ERR_SHAPE, "NVFP4 weight needs N a positive multiple of 8 and K of 32 (N=%lld K=%lld)", (long long)N, (long long)K);
    if (N > (1LL << 30) || K > (1LL << 30)) return fail(ctx, MPQ_ERR_UNSUPPORTED, "dimension above 2^30");
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    mpq_weight* w = new (std::nothrow) mpq_weight();
    if (!w) return fail(ctx, MPQ_ERR_CUDA, "out of host memory");
    w->magic = W_MAGIC;
    w->fmt = MPQ_FMT_NVFP4;
    w->device = ctx->device;
    std::string err;
    int launches = 0;
    int32_t st = nvfp4_weight_build(w->fp4, N, K, codes_host, sf_host, tensor_scale, &launches, err);
    ctx->launches += launches;
    if (st) {
        w->fp4.release();
        delete w;
        return fail(ctx, st, "%s", err.c_str());
    }
    *out = w;
    return MPQ_OK;
}

extern "C" int32_t mpq_nvfp4_gemm_forward(mpq_context* ctx, const mpq_weight* w, const uint8_t* a_codes_dev,
                                          const uint8_t* a_sf_dev, float a_tensor_scale, int64_t M, uint16_t* c_bf16_dev,
                                          void* stream)
{
    if (!ctx_ok(ctx)) return MPQ_ERR_INVALID_ARG;
    if (!w_ok(w) || !a_codes_dev || !a_sf_dev || !c_bf16_dev) return fail(ctx, MPQ_ERR_INVALID_ARG, "null or stale handle / pointer");
    if (w->fmt != MPQ_FMT_NVFP4) return fail(ctx, MPQ_ERR_INVALID_ARG, "weight is not NVFP4");
    if (w->device != ctx->device) return fail(ctx, MPQ_ERR_INVALID_ARG, "weight lives on device %d, context on %d", w->device, ctx->device);
    if (M <= 0 || M > (1LL << 30)) return fail(ctx, MPQ_ERR_SHAPE, "NVFP4 GEMM needs 1 <= M <= 2^30 (M=%lld)", (long long)M);
    if (!aligned16(a_codes_dev) || !aligned16(a_sf_dev) || !aligned16(c_bf16_dev)) return fail(ctx, MPQ_ERR_ALIGN, "A, SFA and C must be 16-byte aligned");
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    std::string err;
    int launches = 0;
    int32_t st = nvfp4_gemm_launch(ctx->fp4, w->fp4, a_codes_dev, a_sf_dev, a_tensor_scale, M, c_bf16_dev,
                                   ctx->prop.multiProcessorCount, (cudaStream_t)stream, &launches, err);
    ctx->launches += launches;
    if (st) return fail(ctx, st, "%s", err.c_str());
    return MPQ_OK;
}

extern "C" int32_t mpq_nvfp4_dequantize(mpq_context* ctx, int64_t R, int64_t K, const uint8_t* codes_dev, const uint8_t* sf_dev,
                                        float tensor_scale, float* out_dev, void* stream)
{
    if (!ctx_ok(ctx)) return MPQ_ERR_INVALID_ARG;
    if (!codes_dev || !sf_dev || !out_dev) return fail(ctx, MPQ_ERR_INVALID_ARG, "null pointer");
    if (R <= 0 || K <= 0 || K % 16) return fail(ctx, MPQ_ERR_SHAPE, "NVFP4 needs K a positive multiple of 16");
    CU_TRY(ctx, cudaSetDevice(ctx->device));
    nvfp4_dequant_launch(codes_dev, sf_dev, tensor_scale, R, K, out_dev, (cudaStream_t)stream);
    ctx->launches += 1;
    CU_TRY(ctx, cudaGetLastError());
    return MPQ_OK;
}
