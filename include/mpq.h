/*
 * libmpq -- block-quantised linear operators for NVIDIA B200 (sm_100a).
 *
 * C ABI.  Every entry point returns an int32 status (0 = MPQ_OK, negative =
 * error), never throws, aborts or prints.  Pointers named *_host are host
 * memory borrowed for the duration of the call; pointers named *_dev are
 * device memory on the context's GPU.  Handles are owned by the library and
 * released by their _destroy call.  "stream" is a cudaStream_t passed as
 * void* (NULL = the legacy default stream); forward calls only enqueue work.
 *
 * Reference interface replaced: none exists.  The makepad/makepad snapshot has
 * no quantised-linear operator, tensor type or CUDA binding; its only AI code
 * is an HTTP chat client (studio/src/ai_chat/ai_chat_manager.rs:778-967).  The
 * shape of this boundary follows the reference's own FFI idiom instead: a
 * run-time loader struct of typed extern "C" function pointers
 * (platform/src/os/linux/module_loader.rs:5-41, egl_sys.rs:311-375), raw
 * pointers plus lengths, #[repr(C)] plain structs (libc_sys.rs:41-44), and an
 * accelerated routine checked against a scalar one (libs/zune-jpeg/src/idct.rs:49-127).
 *
 * Canonical (interchange) formats
 *   Q4     codes  u8[N][K/2]    element 2j = low nibble of byte j, 2j+1 = high
 *                               nibble; nibble = two's-complement int4 in [-8,7]
 *          scales u16[N][K/32]  IEEE binary16 bits; block b covers k in [32b,32b+32)
 *          value  w[n,k] = fp32(scale[n,k/32]) * fp32(code[n,k])     (exact in fp32)
 *   NVFP4  codes  u8[R][K/2]    same nibble order; nibble = e2m1 (S.EE.M)
 *          sf     u8[R][K/16]   e4m3 finite-only bits, non-negative
 *          value  v[r,k] = fp32(e2m1) * fp32(e4m3) * tensor_scale
 */
#ifndef MPQ_H
#define MPQ_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MPQ_OK                  0
#define MPQ_ERR_INVALID_ARG    -1   /* null pointer, bad enum, bad handle */
#define MPQ_ERR_SHAPE          -2   /* K not a multiple of the block size, sizes <= 0, shard does not divide */
#define MPQ_ERR_ALIGN          -3   /* device pointer not 16-byte aligned */
#define MPQ_ERR_CUDA           -4   /* a CUDA runtime/driver call failed; see mpq_last_error */
#define MPQ_ERR_UNSUPPORTED    -5   /* device is not sm_100, or size beyond a stated maximum */
#define MPQ_ERR_PEER_TIMEOUT   -6   /* a bounded device-side wait on a peer flag ran out */
#define MPQ_ERR_STATE          -7   /* call order violated (e.g. exchange used before peers were attached) */
#define MPQ_ERR_FORMAT         -8   /* file is not a weight container this build can use (magic, version, layout, checksum) */
#define MPQ_ERR_IO             -9   /* file cannot be opened, read or written */

#define MPQ_FMT_Q4     1
#define MPQ_FMT_NVFP4  2

#define MPQ_TP_NONE    0
#define MPQ_TP_COLUMN  1   /* split output rows N of W (the columns of W^T) across ranks */
#define MPQ_TP_ROW     2   /* split the reduction dimension K across ranks; partial outputs are summed */

typedef struct mpq_context mpq_context;
typedef struct mpq_weight mpq_weight;
typedef struct mpq_exchange mpq_exchange;

typedef struct mpq_device_info {
    int32_t device;
    int32_t sm_count;
    int32_t cc_major, cc_minor;
    int64_t l2_bytes;
    int64_t total_mem_bytes;
    int32_t sm_clock_khz, mem_clock_khz;
} mpq_device_info;

/* ---- context ------------------------------------------------------------ */
/* One per (process, GPU).  Fails with MPQ_ERR_UNSUPPORTED on anything but
 * compute capability 10.x: there is no fallback path. */
int32_t mpq_context_create(int32_t device, mpq_context** out);
int32_t mpq_context_destroy(mpq_context* ctx);
int32_t mpq_context_info(const mpq_context* ctx, mpq_device_info* out);
const char* mpq_status_string(int32_t status);
/* Text of the last error recorded on this context (thread-compatible, not thread-safe). */
const char* mpq_last_error(const mpq_context* ctx);
/* Reads the device-side status words (this synchronises with all prior work on
 * the GPU): the Q4 and NVFP4 kernels' and, once mpq_q4_linear_forward_static
 * has run on this device, the one inside its static array.
 * MPQ_ERR_PEER_TIMEOUT if a bounded wait inside a kernel ran out since the
 * last poll; the word is then cleared. */
int32_t mpq_context_poll_status(mpq_context* ctx);
/* Number of kernels this context has launched since creation. */
int64_t mpq_context_launch_count(const mpq_context* ctx);

/* ---- Q4 weights ---------------------------------------------------------- */
/* Uploads the canonical arrays and repacks them on the GPU into the layout the
 * kernels stream (16x64 tiles, one 16-byte word group per lane).  With
 * tp_mode COLUMN the handle keeps rows [rank*N/world, (rank+1)*N/world); with
 * ROW it keeps K-slice [rank*K/world, (rank+1)*K/world) (K/world must be a
 * multiple of 32).  Pass tp_mode NONE, rank 0, world 1 for the whole matrix. */
int32_t mpq_q4_weight_create(mpq_context* ctx, int64_t N, int64_t K,
                             const uint8_t* codes_host, const uint16_t* scales_host,
                             int32_t tp_mode, int32_t rank, int32_t world, mpq_weight** out);
/* Same, from canonical arrays already on the device. */
int32_t mpq_q4_weight_create_dev(mpq_context* ctx, int64_t N, int64_t K,
                                 const uint8_t* codes_dev, const uint16_t* scales_dev, mpq_weight** out);

/* ---- NVFP4 weights ------------------------------------------------------- */
/* B is given as [N][K/2] codes (K contiguous per output column) and [N][K/16]
 * e4m3 scales.  K must be a multiple of 32, N a multiple of 8. */
int32_t mpq_nvfp4_weight_create(mpq_context* ctx, int64_t N, int64_t K,
                                const uint8_t* codes_host, const uint8_t* sf_host,
                                float tensor_scale, mpq_weight** out);

/* ---- any weight ---------------------------------------------------------- */
int32_t mpq_weight_shape(const mpq_weight* w, int64_t* N, int64_t* K, int32_t* fmt);
/* Exact fp32 export [N][K] read back FROM THE DEVICE LAYOUT (the bit-exact
 * criterion: proves the repack preserved every value): the Q4 tile stream,
 * or the NVFP4 codes with the scale factors un-tiled from the order the GEMM
 * consumes (the device keeps no other copy of them). */
int32_t mpq_weight_dequantize(mpq_context* ctx, const mpq_weight* w, float* out_dev, void* stream);
int64_t mpq_weight_device_bytes(const mpq_weight* w);
int32_t mpq_weight_destroy(mpq_weight* w);

/* ---- Q4 linear ----------------------------------------------------------- */
/* Forward calls on one context share that context's scratch buffers: issue
 * them in stream order (one stream per context at a time).
 * Y[M][N] = X[M][K] . W^T, fp32 in, fp32 accumulate, fp32 out.  X and Y are
 * row-major device arrays, 16-byte aligned.  Any M >= 1: one row, and up to
 * four rows while M * K < 16384, is one launch of the streaming kernel; up to
 * 16 rows otherwise one pass of the rectangle kernel (weights read once,
 * only a K slice of x staged per CTA) plus a small reduction; from 17 rows slabs of up to 64
 * rows through the tcgen05 kernel (activation staging, main kernel, reduction
 * of the pieces).  The first call that needs a scratch buffer (or a larger
 * one) allocates it: make a warm-up call with the largest M before capturing
 * a CUDA graph.  Finite inputs with |x| < 3e38 are handled at any magnitude
 * (rows are renormalised by a power of two); a non-finite x yields non-finite
 * outputs in its row. */
int32_t mpq_q4_linear_forward(mpq_context* ctx, const mpq_weight* w, const float* x_dev, int64_t M,
                              float* y_dev, void* stream);
/* Same result as mpq_q4_linear_forward for callers that must not let the
 * library allocate (no counterpart in the reference; added for hosts that run
 * inside a fixed memory budget or on a thread that may not enter the CUDA
 * allocator): this call and everything under it performs no cudaMalloc,
 * cudaFree or other allocating routine.  The scratch the M <= 4 kernel needs
 * -- slots for output tiles shared between CTAs -- is a 1 MiB static device
 * array inside the library (512 CTAs' worth; every GPU that loads the library
 * holds it until exit).  A launch that would need more slots is rejected with
 * MPQ_ERR_UNSUPPORTED.  All calls on one device share that array: they must be
 * ordered on the GPU (calls that overlap there race on the slots).  The slots
 * are empty again after every completed call, so nothing needs clearing
 * between calls.  If a bounded wait ran out, slots may be left full: with a
 * status_dev the caller sees it there and must not use this entry point again
 * on that device in this process; without one the kernel records it in a word
 * of the static array that mpq_context_poll_status reads (and, on a timeout,
 * clears together with the slots -- that poll may copy, but allocates nothing).
 * The first call on a device looks up the array's device
 * address and raises the kernels' shared-memory limit; make that call before
 * any stream capture.  status_dev, if not NULL, is a caller-owned device int
 * that a kernel sets non-zero when one of its bounded waits runs out. */
int32_t mpq_q4_linear_forward_static(mpq_context* ctx, const mpq_weight* w, const float* x_dev, int64_t M,
                                     float* y_dev, int32_t* status_dev, void* stream);
/* Convenience end-to-end call with HOST buffers: copies X up, runs, copies Y
 * back and synchronises. */
int32_t mpq_q4_linear_forward_host(mpq_context* ctx, const mpq_weight* w, const float* x_host, int64_t M,
                                   float* y_host);

/* ---- tensor parallelism --------------------------------------------------- */
/* One process per GPU.  A COLUMN shard (mpq_q4_weight_create with MPQ_TP_COLUMN)
 * needs no exchange: each rank's mpq_q4_linear_forward yields its slice of the
 * output columns.  A ROW shard yields a partial output that must be summed
 * over the ranks; the exchange below lets the kernel do that itself, through
 * plain peer stores over NVLink, with no collective library in the data path.
 *
 * An exchange is a buffer on every rank that all ranks can write.  Create it
 * on each rank, pass every rank's 64-byte IPC handle to every other rank (any
 * host transport), and attach.  max_floats bounds M*N of the calls that use it.
 * Single-process users holding peer-mapped pointers attach those directly. */
int32_t mpq_exchange_create(mpq_context* ctx, int32_t rank, int32_t world, int64_t max_floats, mpq_exchange** out);
int32_t mpq_exchange_ipc_handle(mpq_exchange* ex, uint8_t* out64);
/* handles: world * 64 bytes, entry r = rank r's handle (the own entry is ignored). */
int32_t mpq_exchange_attach(mpq_exchange* ex, const uint8_t* handles);
/* buffers[r] = device pointer to rank r's exchange buffer as mapped in this process (own entry ignored). */
int32_t mpq_exchange_attach_pointers(mpq_exchange* ex, void* const* buffers);
int32_t mpq_exchange_buffer(mpq_exchange* ex, void** dev_ptr, int64_t* bytes);
/* Polls a rank waits for one element of a peer's partial output before it gives up,
 * records MPQ_ERR_PEER_TIMEOUT in the context's status word and returns (default 2^22). */
int32_t mpq_exchange_set_wait_limit(mpq_exchange* ex, uint32_t polls);
/* Call after ending a stream capture that recorded calls on this exchange: MPQ_ERR_STATE
 * if the captured graph holds an odd number of them (such a graph must not be replayed,
 * see below), MPQ_OK otherwise.  Clears the condition.  Without this call the next
 * forward call on the exchange reports the same condition. */
int32_t mpq_exchange_graph_check(mpq_exchange* ex);
int32_t mpq_exchange_destroy(mpq_exchange* ex);
/* Row-parallel linear with the sum over ranks fused into the kernel:
 * Y[M][N] = sum_r X_r[M][K/world] . W_r^T on every rank.  Every rank must make the
 * same sequence of calls on the exchange.  Consecutive calls alternate between the
 * two halves of the buffer; a CUDA graph that is replayed must therefore contain an
 * EVEN number of calls on one exchange.  After MPQ_ERR_PEER_TIMEOUT the exchange's
 * contents are undefined: destroy it.  M <= 4 (MPQ_ERR_UNSUPPORTED otherwise: run
 * mpq_q4_linear_forward and reduce with a collective library instead). */
int32_t mpq_q4_linear_forward_allreduce(mpq_context* ctx, const mpq_weight* w, mpq_exchange* ex,
                                        const float* x_dev, int64_t M, float* y_dev, void* stream);

/* ---- SwiGLU between the gate+up and the down projection ------------------- */
/* out[M][F] = silu(gate) * up for gate_up[M][2F] = [gate | up], fp32: silu(g) = g / (1 + exp(-g)) with a
 * correctly rounded division.  F must be a multiple of 4; 16-byte aligned pointers. */
int32_t mpq_swiglu(mpq_context* ctx, const float* gate_up_dev, int64_t M, int64_t F, float* out_dev, void* stream);
/* Y[M][N] = swiglu(gate_up)[M][K] * W^T with gate_up[M][2K]: the down projection with the SwiGLU fused into
 * the kernel's activation staging where mpq_q4_linear_forward would use the streaming kernel (one row, or
 * up to four rows of a short K: the intermediate never exists in memory); otherwise mpq_swiglu runs into
 * scratch the context owns, then mpq_q4_linear_forward.  Same bits as the two calls. */
int32_t mpq_q4_linear_forward_swiglu(mpq_context* ctx, const mpq_weight* w, const float* gate_up_dev, int64_t M,
                                     float* y_dev, void* stream);

/* ---- NVFP4 GEMM ---------------------------------------------------------- */
/* C[M][N] (bf16 bits, row-major) = bf16( tsA * tsB * sum_k A~[m,k] * B~[n,k] ).
 * A is canonical NVFP4 on the device: codes [M][K/2], sf [M][K/16]; any
 * M >= 1.  When K is a multiple of 256 the kernel reads the activation scale
 * factors straight from that array; otherwise they are first re-tiled on the
 * GPU inside this call (counted in its time) into scratch the context owns.
 * C must not overlap A (it is written with TMA tile stores while other tiles
 * are still being read). */
int32_t mpq_nvfp4_gemm_forward(mpq_context* ctx, const mpq_weight* w,
                               const uint8_t* a_codes_dev, const uint8_t* a_sf_dev, float a_tensor_scale,
                               int64_t M, uint16_t* c_bf16_dev, void* stream);
/* Quantises activations to canonical NVFP4 on the GPU, ready to be the GEMM's A: X[M][K] fp32 (or
 * bf16 bits when x_is_bf16 != 0) -> codes [M][K/2], sf [M][K/16].  Per 16-element block the scale
 * byte is e4m3(amax / (6 * tensor_scale)) and each element e2m1(x / (scale * tensor_scale)), both
 * round-to-nearest-even and saturating; a block whose scale encodes to 0 gets zero codes.  K must
 * be a multiple of 16; non-finite inputs are not supported. */
int32_t mpq_nvfp4_quantize_activations(mpq_context* ctx, const void* x_dev, int32_t x_is_bf16, int64_t M, int64_t K,
                                       float tensor_scale, uint8_t* codes_dev, uint8_t* sf_dev, void* stream);
/* The same with SwiGLU fused in front: gate_up[M][2F] = [gate | up] (fp32, or bf16 bits) -> NVFP4 of
 * h = silu(gate) * up (computed in fp32 exactly as mpq_swiglu does; h itself is never written to memory).
 * F must be a multiple of 16.  No counterpart in the reference. */
int32_t mpq_nvfp4_quantize_swiglu(mpq_context* ctx, const void* gate_up_dev, int32_t x_is_bf16, int64_t M, int64_t F,
                                  float tensor_scale, uint8_t* codes_dev, uint8_t* sf_dev, void* stream);
/* Exact fp32 export [R][K] of a canonical NVFP4 tensor on the device. */
int32_t mpq_nvfp4_dequantize(mpq_context* ctx, int64_t R, int64_t K, const uint8_t* codes_dev,
                             const uint8_t* sf_dev, float tensor_scale, float* out_dev, void* stream);

/* ---- weight container ------------------------------------------------------- */
/* Files of two kinds, one 128-byte versioned header + payload + FNV-1a checksum each:
 *   MPQ_FILE_CANONICAL  the interchange arrays (Q4: codes + fp16 scale bits; NVFP4: codes + e4m3 scales +
 *                       tensor scale), readable by any build;
 *   MPQ_FILE_DEVICE     a weight exactly as it lies in device memory (Q4 tile stream; NVFP4 codes + tiled
 *                       scale factors), so that loading needs no repack pass.  It is a CACHE: a file whose
 *                       layout version or geometry is not this build's is refused with MPQ_ERR_FORMAT and
 *                       the caller rebuilds the weight from its canonical arrays (the reference keeps its
 *                       compiled shader binaries the same way, platform/src/os/linux/opengl.rs:611-640).
 * mpq_canonical_* need no GPU.  scales_host is uint16[N][K/32] for Q4, uint8[N][K/16] for NVFP4. */
#define MPQ_FILE_CANONICAL 1
#define MPQ_FILE_DEVICE    2
typedef struct mpq_file_info_t {
    int32_t kind, fmt, layout_version, reserved;
    int64_t N, K;
    int64_t bytes_a, bytes_b;      /* canonical: codes, scales; device: the layout's two buffers */
    float tensor_scale;
    int32_t reserved2;
} mpq_file_info_t;
int32_t mpq_file_info(const char* path, mpq_file_info_t* out);
int32_t mpq_canonical_save(const char* path, int32_t fmt, int64_t N, int64_t K, const uint8_t* codes_host,
                           const void* scales_host, float tensor_scale);
int32_t mpq_canonical_load(const char* path, uint8_t* codes_host, int64_t codes_capacity, void* scales_host,
                           int64_t scales_capacity, float* tensor_scale);
int32_t mpq_weight_save(mpq_context* ctx, const mpq_weight* w, const char* path);
int32_t mpq_weight_load(mpq_context* ctx, const char* path, mpq_weight** out);

/* ---- measured ceilings ------------------------------------------------------ */
/* Probes for whoever reports roofline fractions of the kernels above (no counterpart in the
 * reference; the caller times them with events on `stream`).
 * mpq_probe_hbm_read streams `bytes` of device memory once, read-only, with the loads the Q4 kernels
 * use (out_dev: a device word that is practically never written).  Use a buffer larger than L2.
 * mpq_probe_fp4_mma has every SM issue mmas_per_sm block-scaled FP4 MMAs of the GEMM's own shape
 * (128 x 224 x 64) back to back from resident operands; *flop_out = the flop the launch executes. */
int32_t mpq_probe_hbm_read(mpq_context* ctx, const void* buf_dev, int64_t bytes, uint32_t* out_dev, void* stream);
int32_t mpq_probe_fp4_mma(mpq_context* ctx, int32_t mmas_per_sm, double* flop_out, void* stream);
/* mpq_probe_f16_mma (synchronous; allocates a small result buffer): `issuers` threads of one CTA per SM (1..4, one per
 * warp, each with its own accumulator) issue mmas_per_issuer tcgen05.mma.kind::f16 of 128 x n_cols x 16 with the A
 * operand in tensor memory, as the Q4 tcgen05 kernel does; *cycles_per_mma = median over SMs of the SM cycles from
 * first issue to completion / all MMAs issued on the SM (the tensor pipe needs n_cols / 2 cycles for one). */
int32_t mpq_probe_f16_mma(mpq_context* ctx, int32_t n_cols, int32_t issuers, int32_t mmas_per_issuer, double* cycles_per_mma);

#ifdef __cplusplus
}
#endif
#endif /* MPQ_H */
