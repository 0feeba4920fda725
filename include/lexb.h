/* liblexb - the C ABI of the sm_100a (B200) backend for lex's `gemm_fp4` operator.
 *
 *   y[m,n] (f32) = x[m,k] (f16) . dequant(wq, ws, wg)^T (+ r[m,n])
 *     wq u8[n,k/2]  two E2M1 codes per byte, even column in the low nibble
 *     ws u8[n,k/16] one E4M3 (OCP e4m3fn) scale per 16 weights
 *     wg f32[n]     one scale per row
 *
 * This is the boundary a Rust `lex-cuda` backend would bind with `extern "C"` in place of
 * its NVRTC + driver path: each entry point names the reference interface it stands in
 * for (paths are relative to the lex-gpu tree).  Every function returns 0 on success and a
 * non-zero lexb_status otherwise, with a message in lexb_last_error(); nothing aborts or
 * panics.  All pointers in signatures are plain C; device memory is referred to through
 * opaque lexb_buffer handles (which can wrap a device pointer the caller already owns).
 * There is no CPU fallback: without a compute-capability-10.x device lexb_open fails.
 */
#ifndef LEXB_H
#define LEXB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define LEXB_API
#else
#define LEXB_API __attribute__((visibility("default")))
#endif

typedef enum lexb_status {
    LEXB_OK = 0,
    LEXB_ERR_ARG = 1,          /* null handle, short buffer, misaligned pointer, wrong binding */
    LEXB_ERR_SHAPE = 2,        /* a shape the operator rejects ("does not divide") */
    LEXB_ERR_CUDA = 3,         /* a CUDA call failed; the message carries its error string */
    LEXB_ERR_UNSUPPORTED = 4,  /* no sm_100 device, or a schedule the device cannot hold */
    LEXB_ERR_DEVICE = 5        /* a kernel reported a failure through the status word */
} lexb_status;

typedef struct lexb_gpu lexb_gpu;           /* lex_cuda::Gpu        crates/lex-cuda/src/device.rs:316-325 */
typedef struct lexb_buffer lexb_buffer;     /* lex_cuda::Buffer     crates/lex-cuda/src/device.rs:257-278 */
typedef struct lexb_pipeline lexb_pipeline; /* lex_cuda::Pipeline   crates/lex-cuda/src/device.rs:281-301 */

/* lex_cuda::DeviceInfo, crates/lex-cuda/src/device.rs:303-310 (+ what a B200 plan needs) */
typedef struct lexb_device_info {
    char name[128];
    int cc_major, cc_minor;
    int sm_count;
    int unified_memory;                     /* always 0: weights are staged across PCIe */
    size_t max_threadgroup_bytes;           /* opt-in dynamic shared memory per block */
    uint64_t recommended_working_set_bytes; /* total device memory, as the reference reports */
    size_t l2_bytes;
} lexb_device_info;

/* Optional schedule override, the counterpart of a `.lx` schedule line
 * (crates/lex-front/lx/gemm_fp4.lx:38-39) and of the LEX_GEMM_CU_* variables
 * (crates/lex-msl/src/gemm.rs:90-135).  Zero fields mean "choose". */
typedef struct lexb_sched {
    uint32_t kernel;  /* 0 auto, 1 matvec (m <= 16), 2 tcgen05 GEMM, 3 two-CTA tcgen05 GEMM,
                       * 4 block-scaled FP4 tensor-core kernel (m <= 32; matmul_q_x arithmetic, never chosen by auto) */
    uint32_t tm;      /* tokens per tile of the GEMM: one-CTA kernel a multiple of 16, <= 256; two-CTA kernel 64, 128,
                       * 256 or 512 (0: the planner prices every size with every K split and takes the cheapest) */
    uint32_t stages;  /* pipeline depth of the GEMM */
    uint32_t kc;      /* K columns of x staged per chunk in the matvec: multiple of 1024 */
    uint32_t w_stages; /* two-CTA GEMM: depth of the ring of decoded W tiles (stages = depth of the x ring); tiles below
                        * 512 tokens keep that ring in tensor memory: at most 8 stages there, more puts it in shared memory */
    uint32_t k_splits; /* two-CTA GEMM: split K this many ways (partials in a workspace the pipeline owns, then summed) */
    uint32_t flags;    /* LEXB_SCHED_* bits */
} lexb_sched;
/* Block-scaled kernel and two-CTA GEMM.  Launches are in order on their stream, as the reference's are
 * (crates/lex-cuda/src/device.rs:629-672): every read waits for the kernel ahead.  The kernel can do
 * better when it knows that nothing in flight writes wq and ws - launched with programmatic stream
 * serialization, it then starts loading them while the kernel ahead of it is still running (x, r and y
 * wait as usual).  It knows in two ways:
 *   - inside one lexb_run_launches / lexb_time_launches call the library proves it from the step list (the
 *     call's first launch waits for all earlier work of the stream; a later step whose wq/ws meet no y of an
 *     earlier step of the call loads them early).  LEXB_SCHED_WEIGHTS_MAY_CHANGE turns that off for a pipeline
 *     whose weights something outside the list (another stream) rewrites;
 *   - LEXB_SCHED_WEIGHTS_CONSTANT is the caller's promise that nothing writes wq/ws while launches of
 *     this pipeline are in flight, for launches made one at a time (lexb_gemm_fp4_launch). */
#define LEXB_SCHED_WEIGHTS_MAY_CHANGE 1u
#define LEXB_SCHED_WEIGHTS_CONSTANT 2u

/* lex_msl::program::Lowered, crates/lex-msl/src/program.rs:44-63: the launch descriptor.
 * `writes` is per binding in the order [x, wq, ws, wg, (r), y] (crates/lex-msl/src/gemm.rs:78-82). */
typedef struct lexb_lowered {
    char entry[96];              /* gemm_fp4[_res]_{m}_{n}_{k}_{bm}_{bn}_{bk}, crates/lex-front/src/syntax.rs:933-939 */
    uint32_t grid, grid2;
    uint32_t threads;
    uint32_t threadgroup_bytes;  /* dynamic shared memory */
    uint32_t nbind;
    uint8_t writes[8];           /* (7 bindings for lexb_matmul_int8_plan with a residual) */
    uint32_t kernel;             /* 1 matvec, 2 tcgen05, 3 two-CTA tcgen05, 4 block-scaled FP4 */
    uint32_t m, n, k, residual;
    uint32_t bm, bn, bk, stages;
    uint32_t k_splits;           /* > 1: a second launch sums the partial products */
    uint64_t scratch_bytes;      /* Lowered::scratch_bytes: the split-K workspace */
} lexb_lowered;

/* lex_cuda::Step, crates/lex-cuda/src/device.rs:314: a pipeline and its buffers in binding
 * order [x, wq, ws, wg, (r), y] (QBuf::bind, crates/lex-rt/src/qwen_run.rs:375-387). */
typedef struct lexb_step {
    const lexb_pipeline* pipeline;
    lexb_buffer* const* buffers;
    uint32_t nbuffers;           /* 5 without residual, 6 with; one more ([xq, xs, ...]) for lexb_matmul_int8_plan */
} lexb_step;

LEXB_API const char* lexb_last_error(void);   /* message of this thread's last failing call */
LEXB_API const char* lexb_version(void);

/* Gpu::open, crates/lex-cuda/src/device.rs:350-404.  Takes a device ordinal (the reference
 * always opens device 0) and uses the device's primary context, so that memory allocated by
 * another runtime in the same process (a collective library's buffers) can be wrapped. */
LEXB_API int lexb_open(int device, lexb_gpu** out);
LEXB_API void lexb_close(lexb_gpu* gpu);
/* Gpu::info, crates/lex-cuda/src/device.rs:424-458 */
LEXB_API int lexb_info(lexb_gpu* gpu, lexb_device_info* out);
/* Launches go to the gpu's own stream (non-blocking: it does not synchronise with the legacy default stream)
 * unless a caller-owned CUDA stream is set.  null = the own stream again; a caller that works on the legacy
 * default stream passes cudaStreamLegacy ((cudaStream_t)0x1), not null. */
LEXB_API int lexb_set_stream(lexb_gpu* gpu, void* cuda_stream);
LEXB_API void* lexb_get_stream(lexb_gpu* gpu);
/* cuCtxSynchronize in Gpu::run_launches, crates/lex-cuda/src/device.rs:668-671 */
LEXB_API int lexb_sync(lexb_gpu* gpu);

/* Gpu::zeroed / upload / write / download / download_at, crates/lex-cuda/src/device.rs:527-627 */
LEXB_API int lexb_alloc(lexb_gpu* gpu, size_t bytes, lexb_buffer** out);          /* contents undefined */
LEXB_API int lexb_zeroed(lexb_gpu* gpu, size_t bytes, lexb_buffer** out);
LEXB_API int lexb_wrap(lexb_gpu* gpu, void* device_ptr, size_t bytes, lexb_buffer** out); /* not owned */
LEXB_API int lexb_free(lexb_buffer* buf);                                          /* Buffer::drop */
LEXB_API void* lexb_buffer_ptr(const lexb_buffer* buf);
LEXB_API size_t lexb_buffer_bytes(const lexb_buffer* buf);                         /* Buffer::len_bytes */
LEXB_API int lexb_upload(lexb_gpu* gpu, lexb_buffer* dst, size_t byte_off, const void* src, size_t bytes);
LEXB_API int lexb_download(lexb_gpu* gpu, const lexb_buffer* src, size_t byte_off, void* dst, size_t bytes);
LEXB_API int lexb_memset(lexb_gpu* gpu, lexb_buffer* dst, int byte, size_t bytes);
/* Page-locked host memory for the per-step activations and results. */
LEXB_API int lexb_host_alloc(size_t bytes, void** out);
LEXB_API int lexb_host_free(void* p);

/* lx_kernels::gemm + Gpu::build_lowered, crates/lex-rt/src/lx_kernels.rs:43-107 and
 * crates/lex-cuda/src/device.rs:475-483: choose the kernel and tiles for a shape.  Nothing is
 * compiled at run time; the kernels are built for sm_100a ahead of time.  Shapes must
 * satisfy n % 128 == 0 and k % 64 == 0 (the tcgen05 GEMMs, chosen for m > 8) or n % 16 == 0 and
 * k % 32 == 0 (the matvec, chosen for m <= 8 and for m <= 16 when the GEMMs cannot take the shape);
 * others are refused with LEXB_ERR_SHAPE, as the `.lx` program refuses extents that do not
 * divide (crates/lex-front/src/syntax.rs:1513-1516). */
LEXB_API int lexb_gemm_fp4_plan(lexb_gpu* gpu, uint32_t m, uint32_t n, uint32_t k, int residual,
                                const lexb_sched* sched_or_null, lexb_pipeline** out);
LEXB_API void lexb_pipeline_free(lexb_pipeline* p);                                /* Pipeline::drop */
LEXB_API int lexb_pipeline_describe(const lexb_pipeline* p, lexb_lowered* out);

/* One Step, asynchronous on the gpu's stream: Gpu::run, crates/lex-cuda/src/device.rs:629-648.
 * Buffers in the order [x, wq, ws, wg, (r), y]; r must be null exactly when the pipeline
 * was planned without a residual. */
LEXB_API int lexb_gemm_fp4_launch(lexb_gpu* gpu, const lexb_pipeline* p, const lexb_buffer* x,
                                  const lexb_buffer* wq, const lexb_buffer* ws, const lexb_buffer* wg,
                                  const lexb_buffer* r_or_null, lexb_buffer* y);
/* New (the reference is single-GPU): the n-sharded launch with the all-gather of y fused into the
 * kernel's epilogue.  This rank owns columns [n0, n0 + n) of a gathered y[m, n_total]; y_of_rank[d]
 * is the address, in this GPU's address space, of rank d's gathered y (its own included) - e.g. the
 * peer pointers of a symmetric-memory allocation.  Every finished 128-byte row segment is stored to
 * all `world` buffers with plain peer stores over NVLink (with split-K, by the reduction launch).
 * The caller synchronises the ranks before anyone reads a gathered y.  Two-CTA GEMM shapes only. */
LEXB_API int lexb_gemm_fp4_launch_gather(lexb_gpu* gpu, const lexb_pipeline* p, const lexb_buffer* x,
                                         const lexb_buffer* wq, const lexb_buffer* ws, const lexb_buffer* wg,
                                         const lexb_buffer* r_or_null, void* const* y_of_rank, uint32_t world,
                                         uint32_t n_total, uint32_t n0);
/* gate and up of one MLP in ONE launch with the step after them fused in: the caller interleaves the rows of
 * the two weight matrices once at load (row 2j = gate row j, row 2j + 1 = up row j: lexb_interleave_rows on
 * wq, ws and wg), plans lexb_gemm_fp4_plan(m, 2 * ffn, k) and launches here; the epilogue forms
 * act[m, ffn] = silu(gate) * up as f16 - what `down` reads (X_DTYPE, crates/lex-rt/src/qwen_run.rs:317-327) -
 * and the f32 [m, 2 * ffn] is never written.  It replaces the three dispatches "matvec gate/up" (twice) and
 * silu_mul of crates/lex-rt/src/qwen_run.rs:3165-3183 (crates/lex-front/lx/silu_mul.lx).  Values: the GEMM's
 * own f32 results, then g * (1 / (1 + exp(-g))) * u in f32 with one rounding per operation, then one
 * rounding to f16.  Two-CTA GEMM shapes only (m > 8, 2 * ffn % 128 == 0, k % 256 == 0), no residual; with a
 * K split the reduction launch applies it. */
LEXB_API int lexb_gemm_fp4_silu_launch(lexb_gpu* gpu, const lexb_pipeline* p, const lexb_buffer* x, const lexb_buffer* wq,
                                       const lexb_buffer* ws, const lexb_buffer* wg, lexb_buffer* act);
/* The same, n-sharded, with the all-gather of the activation fused in (no reference counterpart): this rank owns
 * interleaved rows [n0, n0 + n) of n_total (so columns [n0/2, (n0 + n)/2) of act[m, n_total/2]) and stores them
 * into every rank's act buffer with plain peer stores; 2 bytes per output element cross NVLink where the f32
 * gate and up would be 8. */
LEXB_API int lexb_gemm_fp4_silu_launch_gather(lexb_gpu* gpu, const lexb_pipeline* p, const lexb_buffer* x, const lexb_buffer* wq,
                                              const lexb_buffer* ws, const lexb_buffer* wg, void* const* act_of_rank,
                                              uint32_t world, uint32_t n_total, uint32_t n0);
/* out row 2j = a row j, out row 2j + 1 = b row j (device to device, asynchronous on the gpu's stream): the
 * load-time step that puts gate and up rows side by side.  No reference counterpart. */
LEXB_API int lexb_interleave_rows(lexb_gpu* gpu, const lexb_buffer* a, const lexb_buffer* b, size_t rows, size_t row_bytes,
                                  lexb_buffer* out);

/* The call a runtime makes per prefill chunk with host activations: copy x from host memory
 * into x_dev, launch, copy y_dev back into y_host, wait.  The weights stay resident, as
 * lex-rt keeps them (Runner::forward_with writes only per-step inputs,
 * crates/lex-rt/src/qwen_run.rs:2348-2373, and downloads the result, :2401-2404). */
LEXB_API int lexb_gemm_fp4_run_host(lexb_gpu* gpu, const lexb_pipeline* p, const void* x_host, lexb_buffer* x_dev,
                                    const lexb_buffer* wq, const lexb_buffer* ws, const lexb_buffer* wg,
                                    const lexb_buffer* r_or_null, lexb_buffer* y_dev, void* y_host);
/* The same three steps enqueued on the gpu's current stream without the wait: the caller calls lexb_sync
 * (on that stream) before it reads y_host or rewrites x_host.  With two streams (lexb_set_stream) and two
 * sets of staging buffers a caller overlaps one chunk's copy back with the next chunk's copy in and launch;
 * the reference has no counterpart (its runtime is synchronous per batch, crates/lex-cuda/src/device.rs:650-672). */
LEXB_API int lexb_gemm_fp4_enqueue_host(lexb_gpu* gpu, const lexb_pipeline* p, const void* x_host, lexb_buffer* x_dev,
                                        const lexb_buffer* wq, const lexb_buffer* ws, const lexb_buffer* wg,
                                        const lexb_buffer* r_or_null, lexb_buffer* y_dev, void* y_host);
/* Gpu::run_launches, crates/lex-cuda/src/device.rs:650-672: all steps, one synchronise;
 * cpu_s = host time to enqueue, wall_s = host time until the device is idle.
 * The results are those of the steps run one after another.  Consecutive lexb_matmul_fp4_plan steps of t <= 8
 * tokens planned with k_splits = 1 (and without LEXB_SCHED_WEIGHTS_MAY_CHANGE), with the same t, k
 * and activation type, of which none reads or overwrites a buffer that an earlier one of them touches (x, r,
 * wq and ws not written, y neither read nor written: the address ranges are compared; wq and ws must also be
 * untouched by every earlier step of the call, or declared constant), are run as ONE persistent kernel
 * over all their row tiles (the gate/up pair, q/k/v); each result is bit-identical to the step launched alone.
 * A step that depends on the run starts a new launch.  The environment variable LEXB_CHAIN=0 turns this off. */
LEXB_API int lexb_run_launches(lexb_gpu* gpu, const lexb_step* steps, size_t nsteps, double* cpu_s, double* wall_s);
/* How lexb_run_launches would issue this list, without launching anything: run_len_out[i] = number of steps of
 * the kernel launch that step i belongs to (1: a launch of its own).  No counterpart in the reference; for
 * callers and tests that want to see which steps share a launch. */
LEXB_API int lexb_list_runs(lexb_gpu* gpu, const lexb_step* steps, size_t nsteps, uint32_t* run_len_out);
/* Gpu::run_each_timed, crates/lex-cuda/src/device.rs:684-739: device seconds per step,
 * from events recorded between launches, no synchronise in between. */
LEXB_API int lexb_run_each_timed(lexb_gpu* gpu, const lexb_step* steps, size_t nsteps, double* seconds_out);
/* Device seconds for `reps` back-to-back passes over the steps (events on the launch stream). */
LEXB_API int lexb_time_launches(lexb_gpu* gpu, const lexb_step* steps, size_t nsteps, uint32_t reps, double* seconds_out);

/* Kernels never spin without a limit: a wait that gives up ORs a code into a device status
 * word and the kernel leaves in order.  This reads the word (after a synchronise) and clears it. */
LEXB_API int lexb_status_word(lexb_gpu* gpu, uint32_t* out);
/* Runs a one-block kernel whose only wait is on a barrier nothing will ever complete, with a
 * limit of `limit_us` microseconds, to show that the bounded wait reports and returns.  Sets
 * the status word to LEXB_STATUS_WAIT_NEVER. */
LEXB_API int lexb_selftest_bounded_wait(lexb_gpu* gpu, uint32_t limit_us);
#define LEXB_STATUS_WAIT_NEVER (1u << 16)

/* In-kernel phase timers of the two-CTA GEMM (the counterpart of LEX_SYNC's per-call-site
 * attribution, crates/lex-rt/src/qwen_run.rs:2926-2960, one level down): with tracing enabled
 * for up to max_ctas blocks, each block of the next launch records 16 SM-clock values:
 * [0] start, [1] first K step ready, [2] all MMAs issued, [3] cycles the MMA warp waited for the
 * inputs of a K step (x tiles and both CTAs' W tiles report to one barrier), [4] and [5] zero,
 * [6] accumulator complete, [7] epilogue done ([1]-[5] and, as [11], the cycles spent issuing MMAs
 * only in the leader block of a pair); [8..10] and [12..14]: for the
 * first and the last dequant thread, cycles in the decode loop, of which waiting for packed
 * weights, of which waiting for a free W stage; [15] the block's end and, in the partner block of a
 * pair, [11] its start, both in nanoseconds of the GPU's global timer.  With max_ctas >= twice the
 * grid, consecutive launches record into alternating halves of the buffer, so that two launches in a
 * row can be read side by side.  max_ctas = 0 turns it off.
 * The block-scaled kernel records, per block: [0] start, [1] first stage ready to multiply, [2] all
 * MMAs issued, [3] cycles its MMA warp waited for codes, [4] for scale blocks and pieces, [5] spent
 * issuing; [6..8] the first scale warp's loop, of which waiting for a free stage, for scale bytes;
 * [9] when its barriers were initialised (low half) and fenced (high half), relative to the start;
 * [10] block done; [11..12] the first piece warp's loop, of which waiting for a free stage;
 * [13] first copy issued, [14] first codes landed, [15] set-up done. */
LEXB_API int lexb_trace_enable(lexb_gpu* gpu, uint32_t max_ctas);
LEXB_API int lexb_trace_read(lexb_gpu* gpu, uint64_t* out, uint32_t ctas);

/* Test hook for the bit-exact claim: the f16 every kernel multiplies by, for all n*k weights,
 * written row-major as u16 bit patterns (the value Op::Stage produces,
 * crates/lex-front/src/interp.rs:500-507, from Op::DequantFp4, :643-657). */
LEXB_API int lexb_dequant_fp4_f16(lexb_gpu* gpu, uint32_t n, uint32_t k, const lexb_buffer* wq,
                                  const lexb_buffer* ws, const lexb_buffer* wg, lexb_buffer* w_f16);

/* No counterpart in the reference.  The split-K form of the two-CTA GEMM for callers that must not
 * allocate device memory once they are running: a runtime that handed the whole device to its own
 * pool at start-up (lex-rt sizes its caches off total device memory, crates/lex-cuda/src/device.rs:449-456),
 * so that a later cudaMalloc for a workspace can fail, or a decode loop that cannot afford the
 * device-wide synchronisation an allocation implies.  lexb_gemm_fp4_plan allocates the split-K
 * workspace; this call instead keeps the partial products in a 32 MiB array that is part of the
 * library image (LEXB_STATIC_SCRATCH_BYTES; every GPU that loads the library holds it until exit), and
 * calls no cudaMalloc / cudaFree or other allocating routine.  It plans and launches in one call:
 * y = x . W^T (+ r) with K split `k_splits` ways (2..8, whole blocks of 256 columns), m >= 128,
 * n % 128 == 0, k % 256 == 0.  Shapes whose partials (splits * m * n * 4 bytes) exceed the array are
 * refused with LEXB_ERR_UNSUPPORTED and a message that says so.
 * The first call on a device resolves the array's device address (cudaGetSymbolAddress); make that
 * first call before any stream capture.  All calls on a device share the array, which keeps the last
 * call's partials: nothing needs clearing (every partial is written before it is read), but two
 * calls that overlap on the GPU - different streams, or different gpu handles of one device - race.
 * Results are bit-identical to a pipeline planned with the same k_splits. */
#define LEXB_STATIC_SCRATCH_BYTES (32ull << 20)
LEXB_API int lexb_gemm_fp4_splitk_static(lexb_gpu* gpu, uint32_t m, uint32_t n, uint32_t k, uint32_t k_splits,
                                         const lexb_buffer* x, const lexb_buffer* wq, const lexb_buffer* ws,
                                         const lexb_buffer* wg, const lexb_buffer* r_or_null, lexb_buffer* y);

/* lex_front::llama::matmul_q_x with the NVFP4 layout (crates/lex-front/src/llama.rs:444-499): the
 * operator the model runs for decode and speculative verification (t <= 8,
 * crates/lex-rt/src/qwen_run.rs:2605-2606), same bindings [x, wq, ws, wg, (r), y] as gemm_fp4 but with
 * the weights used as dequantised f32 values (e2m1 * e4m3 * wg, crates/lex-front/src/interp.rs:643-657),
 * not rounded to f16.  The pipeline is launched like any other (lexb_gemm_fp4_launch, lexb_step).
 * Here: t <= 32 tokens, activations f16 (x_half != 0) or f32 (x_half == 0), n_out % 128 == 0,
 * n_in % 256 == 0.  The decode runs on the tensor cores' block-scaled FP4 path, which takes wq and ws
 * as stored; each token is split into eight rows of 2-bit E2M1 digits: 16 significant bits below the
 * largest value of every group of 16, exact for f16 values within 2^5 of that maximum, and for f32
 * input the precision the reference's integer path keeps (quant16, crates/lex-msl/src/int8.rs:44-99).
 * Results agree with the interpreter to about 1e-5 of scale (gate 2e-3,
 * crates/lex-cuda/tests/device_gpu.rs:294-303); the entry name is the reference's
 * (matvec_nvfp4_{n_out}x{n_in}[_res][_xh], matmul{t}_... for t > 1).  A token holding an infinity or a
 * NaN gives NaN for the whole token; magnitudes below 2^-111 count as zero. */
LEXB_API int lexb_matmul_fp4_plan(lexb_gpu* gpu, uint32_t t, uint32_t n_out, uint32_t n_in, int residual, int x_half,
                                  const lexb_sched* sched_or_null, lexb_pipeline** out);

/* lex_msl::int8 (crates/lex-msl/src/int8.rs): the integer-activation path the reference decodes and verifies with
 * on CUDA for t <= 4 tokens (crates/lex-rt/src/qwen_run.rs:2876-2924).
 * lexb_quant16 = int8::quant16 (:47-114), operation for operation: each group of 16 values of x[m, k] (f32, or f16
 * when x_half) becomes 16 int16 in xq[m, k] and one f32 scale in xs[m, k/16] (largest magnitude / 32767); k % 32 == 0.
 * lexb_matmul_int8_plan = int8::matmul_int8 (:121-223): y[t, n] = sum_p (xq * xs)[t, p] * W[n, p] (+ r) with the NVFP4
 * W as matmul_q_x takes it; the pipeline is launched as a lexb_step with the reference's bindings
 * [xq, xs, wq, ws, wg, (r), y] (7 with the residual).  Here the products run on the block-scaled FP4 tensor-core
 * kernel (t <= 32, n % 128 == 0, k % 256 == 0): the activation is widened to xq * xs in f32 and split into digit
 * rows like any f32 activation, which keeps 16 bits below each group's largest value - the precision int16
 * carries.  Within the reference's bar for this path against the interpreter's matmul_q_x (2e-3 of scale,
 * crates/lex-cuda/tests/device_gpu.rs:314-380), and a token's result does not depend on its batch. */
LEXB_API int lexb_quant16(lexb_gpu* gpu, uint32_t m, uint32_t k, int x_half, const lexb_buffer* x, lexb_buffer* xq,
                          lexb_buffer* xs);
LEXB_API int lexb_matmul_int8_plan(lexb_gpu* gpu, uint32_t t, uint32_t n_out, uint32_t n_in, int residual,
                                   const lexb_sched* sched_or_null, lexb_pipeline** out);

/* The step after gate/up in the MLP: out = silu(gate) * up, elementwise in f32, written as f16 (what
 * `down` reads, X_DTYPE in crates/lex-rt/src/qwen_run.rs:317-327) or f32.  The operator is
 * crates/lex-front/lx/silu_mul.lx / lex_front::llama::silu_mul (crates/lex-front/src/llama.rs:858-891).
 * gate and up are f32 [rows, cols] views given by a buffer, an offset and a row pitch in elements, so
 * that one gemm_fp4 launch over gate's and up's rows concatenated ([m, 2n] output) feeds it directly:
 * gate = (y, 0, 2n), up = (y, n, 2n). */
LEXB_API int lexb_silu_mul(lexb_gpu* gpu, uint32_t rows, uint32_t cols, const lexb_buffer* gate, size_t gate_offset,
                           size_t gate_pitch, const lexb_buffer* up, size_t up_offset, size_t up_pitch,
                           lexb_buffer* out, int out_f16);

/* Runner::chunk / prefill_limit, crates/lex-rt/src/qwen_run.rs:2478-2501 with GEMM_SIZES and MAX_BATCH of
 * :730-746: how a prompt of `tokens` is cut into prefill chunks - the largest of 512, 256, 128, 64, 32, 16
 * that fits under `limit` (0 = 512) and the tokens left, then at most 8 at a time for the batched
 * matvec.  gemm_ok = 0 reproduces the no-GEMM fallback (chunks of 8).  chunks may be null to count. */
LEXB_API int lexb_prefill_chunks(uint32_t tokens, uint32_t limit, int gemm_ok, uint32_t* chunks, uint32_t max_chunks,
                                 uint32_t* count);

/* Host-side failure injection, for tests of the error paths: the nth call from now (1 = the next) that
 * reaches `site` is not made and reports `cuda_error` (a cudaError_t value; 0 = cudaErrorUnknown) instead, so
 * that the entry point around it returns LEXB_ERR_CUDA, releases what it had taken and leaves its handles
 * usable.  Sites: 1 device allocation, 2 host<->device copy, 3 kernel launch, 4 tensor-map encoding;
 * site 0 disarms everything.  Nothing on the device is made to fail.  It stands in for the injectable
 * driver table of the reference (the `api!` table, crates/lex-cuda/src/device.rs:88-132). */
#define LEXB_SITE_ALLOC 1
#define LEXB_SITE_COPY 2
#define LEXB_SITE_LAUNCH 3
#define LEXB_SITE_ENCODE 4
LEXB_API int lexb_debug_fail_next(int site, int nth, int cuda_error);

/* Column-parallel sharding over `world` devices (new: the reference is single-GPU,
 * crates/lex-cuda/src/device.rs:358-359).  Rank `rank` owns weight rows [*n0, *n1) - whole
 * 128-row tiles, the remainder spread over the first ranks - of wq, ws and wg, and writes the
 * same columns of y. */
LEXB_API int lexb_shard_rows(uint32_t n, uint32_t world, uint32_t rank, uint32_t* n0, uint32_t* n1);

#ifdef __cplusplus
}
#endif
#endif /* LEXB_H */
