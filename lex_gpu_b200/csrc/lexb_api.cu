// Host side of liblexb: the C ABI declared in include/lexb.h over the CUDA runtime.
// It mirrors lex_cuda::device (crates/lex-cuda/src/device.rs): a Gpu that owns a stream,
// Buffers, Pipelines (a planned kernel + launch shape) and Steps, with string errors
// instead of panics.  Kernels are compiled ahead of time for sm_100a and live in this
// library; there is no NVRTC step and no CPU path.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <map>
#include <string>
#include <tuple>
#include <unordered_map>
#include <vector>

#include "../../include/lexb.h"
#include "gemm_fp4_sm100.cuh"
#include "gemm_fp4_sm100_pair.cuh"
#include "matvec_fp4_sm100.cuh"
#include "matmul_q_fp4_sm100.cuh"
#include "matmul_q_chain_sm100.cuh"

// Scratch of lexb_gemm_fp4_splitk_static: split-K partial products [splits][m][n] f32.  Part of
// the library image, so every GPU that loads the library holds these 32 MiB until the process exits.
static __device__ __align__(256) float g_splitk_static_scratch[LEXB_STATIC_SCRATCH_BYTES / sizeof(float)];

namespace {

thread_local std::string g_last_error;
thread_local bool t_injected = false;     // the failure being reported was made by lexb_debug_fail_next

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    if (t_injected) g_last_error += " [injected]";
    t_injected = false;
    return code;
}

#define CUDA_TRY(expr)                                                                          \
    do {                                                                                        \
        cudaError_t e_ = (expr);                                                                \
        if (e_ != cudaSuccess)                                                                  \
            return fail(LEXB_ERR_CUDA, "%s: %s (%s)", #expr, cudaGetErrorString(e_), cudaGetErrorName(e_)); \
    } while (0)

// Host-side failure injection (tests only): lexb_debug_fail_next arms one site; the n-th call that reaches it
// from then on fails with the given CUDA error instead of being made.  It stands where the reference's
// injectable driver table would (the `api!` table, crates/lex-cuda/src/device.rs:88-132); nothing on the
// device is made to fail.
enum { SITE_ALLOC = 1, SITE_COPY = 2, SITE_LAUNCH = 3, SITE_ENCODE = 4, SITE_COUNT = 5 };
struct Injection { int countdown = 0; int error = 0; };
Injection g_inject[SITE_COUNT];
std::mutex g_inject_lock;

cudaError_t take_injected(int site) {
    std::lock_guard<std::mutex> lk(g_inject_lock);
    Injection& in = g_inject[site];
    if (in.countdown > 0 && --in.countdown == 0) {
        t_injected = true;
        return static_cast<cudaError_t>(in.error);
    }
    return cudaSuccess;
}

#define CUDA_TRY_AT(site, expr)                                                                 \
    do {                                                                                        \
        cudaError_t e_ = take_injected(site);                                                   \
        if (e_ == cudaSuccess) e_ = (expr);                                                     \
        if (e_ != cudaSuccess)                                                                  \
            return fail(LEXB_ERR_CUDA, "%s: %s (%s)", #expr, cudaGetErrorString(e_), cudaGetErrorName(e_)); \
    } while (0)
#define LAUNCH_TRY(expr) CUDA_TRY_AT(SITE_LAUNCH, expr)
// in front of a <<<...>>> launch
#define INJECT_LAUNCH()                                                                         \
    do {                                                                                        \
        if (cudaError_t e_ = take_injected(SITE_LAUNCH))                                        \
            return fail(LEXB_ERR_CUDA, "kernel launch: %s (%s)", cudaGetErrorString(e_), cudaGetErrorName(e_)); \
    } while (0)

cudaError_t x_malloc(void** p, size_t bytes) {
    if (cudaError_t e = take_injected(SITE_ALLOC)) { *p = nullptr; return e; }
    return cudaMalloc(p, bytes);
}
template <typename T> cudaError_t x_malloc(T** p, size_t bytes) { return x_malloc(reinterpret_cast<void**>(p), bytes); }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

enum { KERNEL_MATVEC = 1, KERNEL_TCGEN05 = 2, KERNEL_TCGEN05_PAIR = 3, KERNEL_MATMUL_Q = 4 };
thread_local bool t_plan_q16 = false;      // set by lexb_matmul_int8_plan around its call of lexb_gemm_fp4_plan

}  // namespace

struct lexb_gpu {
    int device = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;       // own_stream or the caller's
    uint32_t* d_status = nullptr;
    bool pdl = true;                         // programmatic dependent launch of the two-CTA GEMM
    float* static_scratch = nullptr;         // device address of g_splitk_static_scratch on this device, once resolved
    // Job tables of chained runs, kept by content: a decode loop issues the same lists token after token, and a
    // table found here needs no copy in front of its launch (a copy would put the launch behind the whole
    // kernel before it).  A table is never written again once copied.
    struct ChainTable { std::vector<lexb::MqChainJob> host; lexb::MqChainJob* dev; };
    std::unordered_multimap<uint64_t, ChainTable> chain_tables;
    // Digit rows of a run's activations (matmul_q_pieces_kernel's output: [8 m][k / 2] digit rows, [k / 256][2048]
    // scale blocks, [m] magnitudes), one buffer per activation buffer, shape and stream: rewritten by every run that
    // reads that x, in stream order.
    struct ChainPre { uint8_t* buf; CUtensorMap map; };
    std::map<std::tuple<const void*, uint32_t, uint32_t, bool, cudaStream_t>, ChainPre> chain_pre;
    unsigned long long* d_trace = nullptr;   // phase timers of the last two-CTA launch, when tracing is on
    size_t trace_ctas = 0;
    uint32_t trace_toggle = 0;
    cudaDeviceProp prop{};
    EncodeTiledFn encode_tiled = nullptr;
    size_t smem_optin = 0;
};

struct lexb_buffer {
    lexb_gpu* gpu;
    void* ptr;
    size_t bytes;
    bool owned;
};

struct lexb_pipeline {
    lexb_gpu* gpu;
    uint32_t kernel;
    uint32_t m, n, k;
    bool residual;
    // tcgen05 GEMM
    uint32_t tm, stages, w_stages, tmem_cols, m_tiles, n_acc, flags;
    uint32_t raw_stages = lexb::PAIR_RAW_STAGES;
    uint32_t k_sub = 1;         // two-CTA kernel: K steps per ring stage
    uint32_t x_rows = lexb::PAIR_XBLK_ROWS;     // two-CTA kernel: tokens per CTA and token block (tm / 2 for tiles below 512 tokens)
    uint32_t k_splits = 1, kb_per_split = 0, tok_blocks = 2;
    uint32_t ws_pitch = 0;      // block-scaled kernel: bytes per row of one scale load
    bool x_f32 = false;         // ... with f32 activations
    bool x_q16 = false;         // ... with int16 activations and one f32 scale per 16 (lexb_matmul_int8_plan): bindings [xq, xs, wq, ...]
    bool w_const = false;       // the caller declared wq/ws constant (LEXB_SCHED_WEIGHTS_CONSTANT): loaded ahead of the stream's order
                                // by the kernels that can (block-scaled kernel, two-CTA GEMM)
    bool w_volatile = false;    // ... or said they may change (LEXB_SCHED_WEIGHTS_MAY_CHANGE): never loaded early, not even in a list
    bool mq_pre = false;        // ... with the tokens' digit rows from the pieces kernel: buffers and their tensor map
    uint8_t* pre_buf = nullptr; // [8 m][k / 2] digit rows, then [k / 256][2048] scale blocks, then [m] magnitudes
    CUtensorMap pre_map{};
    float* partial = nullptr;   // split-K workspace [k_splits][m][n], owned by the pipeline
    // matvec
    uint32_t kc;
    uint32_t grid, threads, smem;
    char entry[96];
    // tensor maps of x, keyed by the device pointer they were encoded for
    struct MapEntry {
        const void *x, *wq, *ws;
        CUtensorMap map, map_wq, map_ws;
    };
    mutable std::vector<MapEntry> maps;
    mutable std::mutex maps_lock;
};

namespace {

int use(lexb_gpu* g) {
    if (!g) return fail(LEXB_ERR_ARG, "null gpu handle");
    CUDA_TRY(cudaSetDevice(g->device));
    return LEXB_OK;
}

int check_buf(const lexb_buffer* b, const lexb_gpu* g, size_t need, const char* what) {
    if (!b) return fail(LEXB_ERR_ARG, "%s: null buffer", what);
    if (b->gpu != g) return fail(LEXB_ERR_ARG, "%s: buffer belongs to another gpu handle", what);
    if (b->bytes < need) return fail(LEXB_ERR_ARG, "%s: buffer holds %zu bytes, the shape needs %zu", what, b->bytes, need);
    if ((reinterpret_cast<uintptr_t>(b->ptr) & 15u) != 0) return fail(LEXB_ERR_ARG, "%s: device pointer is not 16-byte aligned", what);
    return LEXB_OK;
}

uint32_t round_up(uint32_t v, uint32_t to) { return (v + to - 1) / to * to; }

uint32_t env_u32(const char* name, uint32_t dflt) {
    const char* s = getenv(name);
    if (!s || !*s) return dflt;
    return static_cast<uint32_t>(strtoul(s, nullptr, 10));
}

// one-block kernel for lexb_selftest_bounded_wait: a barrier with one expected arrival that
// never comes; the wait gives up after limit_cycles and reports.
__global__ void bounded_wait_selftest_kernel(uint32_t* status, long long limit_cycles) {
    __shared__ __align__(8) uint64_t bar;
    const uint32_t b = lexb::smem_u32(&bar);
    if (threadIdx.x == 0) {
        lexb::mbar_init(b, 1);
        lexb::fence_mbar_init();
        const long long t0 = clock64();
        bool done = false;
        while (!(done = lexb::mbar_try_wait(b, 0))) {
            if (clock64() - t0 > limit_cycles) break;
        }
        if (!done) atomicOr(status, lexb::ST_WAIT_NEVER);
    }
}

// every staged weight as f16 bits: one thread per group of 16
__global__ void dequant_fp4_f16_kernel(uint32_t n, uint32_t k, const uint8_t* __restrict__ wq,
                                       const uint8_t* __restrict__ ws, const float* __restrict__ wg,
                                       uint16_t* __restrict__ out) {
    const uint32_t groups_per_row = k / 16u;
    const size_t total = static_cast<size_t>(n) * groups_per_row;
    for (size_t gi = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; gi < total;
         gi += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint32_t row = static_cast<uint32_t>(gi / groups_per_row);
        const uint2 q = *reinterpret_cast<const uint2*>(wq + gi * 8u);
        uint4 lo, hi;
        lexb::decode_group16(q, ws[gi], wg[row], lo, hi);
        uint4* o = reinterpret_cast<uint4*>(out + gi * 16u);
        o[0] = lo;
        o[1] = hi;
    }
}

// a = silu(g) * u = g * (1 / (1 + exp(-g))) * u, evaluated in f32 in that order
// (crates/lex-front/src/llama.rs:879-888, sigmoid as crates/lex-front/src/ir.rs:244), four columns per thread.
template <typename OutT>
__global__ void silu_mul_kernel(uint32_t rows, uint32_t cols, const float* __restrict__ g, size_t g_pitch,
                                const float* __restrict__ u, size_t u_pitch, OutT* __restrict__ out) {
    const uint32_t c4 = cols / 4u;
    const size_t total = static_cast<size_t>(rows) * c4;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t r = i / c4, c = (i - r * c4) * 4u;
        const float4 gv = *reinterpret_cast<const float4*>(g + r * g_pitch + c);
        const float4 uv = *reinterpret_cast<const float4*>(u + r * u_pitch + c);
        const float gg[4] = {gv.x, gv.y, gv.z, gv.w}, uu[4] = {uv.x, uv.y, uv.z, uv.w};
        float y[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            y[j] = lexb::silu_mul_f32(gg[j], uu[j]);
        }
        if constexpr (sizeof(OutT) == 4) {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + r * cols + c) = make_float4(y[0], y[1], y[2], y[3]);
        } else {
            uint2 packed;
            packed.x = lexb::pack_f16x2_rn(y[0], y[1]);
            packed.y = lexb::pack_f16x2_rn(y[2], y[3]);
            *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(out) + r * cols + c) = packed;
        }
    }
}

// lex_msl::int8::quant16 (crates/lex-msl/src/int8.rs:47-114), operation for operation: per group of 16 the largest
// magnitude mx, inv = 32767 / mx (0 for a group of zeros), q = round-to-nearest-even(v * inv) as int16, scale mx / 32767.
template <bool XH>
__global__ void quant16_kernel(const void* __restrict__ x, short* __restrict__ xq, float* __restrict__ xs, size_t groups) {
    const size_t g = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (g >= groups) return;
    float v[16];
    if (XH) {
        const uint4* xp = reinterpret_cast<const uint4*>(x) + g * 2u;
        const uint4 raw[2] = {xp[0], xp[1]};
        const __half2* hp = reinterpret_cast<const __half2*>(raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 f = __half22float2(hp[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    } else {
        const float4* xp = reinterpret_cast<const float4*>(x) + g * 4u;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 f = xp[i];
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
    }
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) mx = fmaxf(mx, fabsf(v[i]));
    const float inv = mx > 0.0f ? __fdiv_rn(32767.0f, mx) : 0.0f;
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
        w[i] = (static_cast<uint32_t>(__float2int_rn(__fmul_rn(v[2 * i], inv))) & 0xFFFFu) |
               ((static_cast<uint32_t>(__float2int_rn(__fmul_rn(v[2 * i + 1], inv))) & 0xFFFFu) << 16);
    uint4* out = reinterpret_cast<uint4*>(xq) + g * 2u;
    out[0] = make_uint4(w[0], w[1], w[2], w[3]);
    out[1] = make_uint4(w[4], w[5], w[6], w[7]);
    xs[g] = __fdiv_rn(mx, 32767.0f);
}

int encode_2d(const lexb_pipeline* p, CUtensorMap* map, CUtensorMapDataType dt, uint32_t esize, const void* ptr,
              uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz,
              const char* what) {
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {inner * esize};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    if (cudaError_t ie = take_injected(SITE_ENCODE))
        return fail(LEXB_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)ie);
    CUresult r = p->gpu->encode_tiled(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LEXB_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
    return LEXB_OK;
}

// Tensor maps for one binding, cached by the device pointers they were encoded for.
int get_maps(const lexb_pipeline* p, const void* x, const void* wq, const void* ws, lexb_pipeline::MapEntry* out) {
    std::lock_guard<std::mutex> lk(p->maps_lock);
    const bool pair = p->kernel == KERNEL_TCGEN05_PAIR || p->kernel == KERNEL_MATMUL_Q;
    for (const auto& e : p->maps)
        if (e.x == x && (!pair || (e.wq == wq && e.ws == ws))) {
            *out = e;
            return LEXB_OK;
        }
    lexb_pipeline::MapEntry e{};
    e.x = x; e.wq = wq; e.ws = ws;
    int rc;
    // x f16[m, k] row-major; box = 64 columns (128 bytes, the swizzle span) x the tile's tokens, never
    // taller than the tensor.  Rows past m are filled with zeros by the copy engine.
    const uint32_t box_rows = pair ? (p->m < p->x_rows ? p->m : p->x_rows) : (p->tm < p->m ? p->tm : p->m);
    if (p->kernel != KERNEL_MATMUL_Q &&      // that kernel reads x with plain loads
        (rc = encode_2d(p, &e.map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x, p->k, p->m, lexb::GEMM_BK, box_rows,
                        CU_TENSOR_MAP_SWIZZLE_128B, "x")))
        return rc;
    if (pair) {
        // wq u8[n, k/2]: 128 rows x 128 bytes (256 columns of K), swizzled; ws u8[n, k/16]: 128 rows x 16 bytes
        if ((rc = encode_2d(p, &e.map_wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, p->k / 2, p->n, lexb::PAIR_RAW_K / 2,
                            lexb::GEMM_TN, CU_TENSOR_MAP_SWIZZLE_128B, "wq")))
            return rc;
        const uint32_t ws_box = p->kernel == KERNEL_MATMUL_Q ? p->ws_pitch : lexb::PAIR_RAW_K / 16;
        if ((rc = encode_2d(p, &e.map_ws, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, ws, p->k / 16, p->n, ws_box,
                            lexb::GEMM_TN, CU_TENSOR_MAP_SWIZZLE_NONE, "ws")))
            return rc;
    }
    if (p->maps.size() >= 64) p->maps.erase(p->maps.begin());
    p->maps.push_back(e);
    *out = e;
    return LEXB_OK;
}

// The weights of the launch that follows in a step list: a hint for the block-scaled kernel, which pulls
// their first stages into L2 before it ends.
struct NextWeights {
    const lexb_pipeline* pipe;
    const lexb_buffer *x, *wq, *ws;
};

// How a launch sits in its stream.  `early_weights`: the block-scaled kernel may load wq/ws before the launch ahead of
// it has finished (the caller declared them constant, or the step list shows that nothing in flight writes them).
// `fence`: launched without programmatic stream serialization, so that it starts only when everything ahead of it
// in the stream is done - the first launch of a step list, behind which the list's own launches overlap one another only.
struct Order {
    bool early_weights = false;
    bool fence = false;
};

int launch_one(lexb_gpu* g, const lexb_pipeline* p, const lexb_buffer* x, const lexb_buffer* wq, const lexb_buffer* ws,
               const lexb_buffer* wg, const lexb_buffer* r, lexb_buffer* y, const lexb::GatherDst* gather = nullptr,
               const NextWeights* next = nullptr, Order order = Order{}, lexb_buffer* act = nullptr,
               const lexb_buffer* xs_q16 = nullptr) {
    const bool pdl = g->pdl && !order.fence;
    // gate/up fused: `act` (or a gather whose destination buffers are f16 activations) replaces y
    const bool silu = act != nullptr || (gather && gather->silu);
    if (!p) return fail(LEXB_ERR_ARG, "null pipeline");
    if (p->gpu != g) return fail(LEXB_ERR_ARG, "pipeline was planned on another gpu handle");
    const size_t m = p->m, n = p->n, k = p->k;
    int rc;
    if ((rc = check_buf(x, g, m * k * (p->x_f32 ? 4 : 2), p->x_q16 ? "xq" : "x"))) return rc;
    if (p->x_q16) {
        if ((rc = check_buf(xs_q16, g, m * (k / 16) * 4, "xs"))) return rc;
    } else if (xs_q16) {
        return fail(LEXB_ERR_ARG, "an activation-scale buffer was bound to a pipeline that takes f16 or f32 activations");
    }
    if ((rc = check_buf(wq, g, n * k / 2, "wq"))) return rc;
    if ((rc = check_buf(ws, g, n * k / 16, "ws"))) return rc;
    if ((rc = check_buf(wg, g, n * 4, "wg"))) return rc;
    if (silu) {
        if (p->kernel != KERNEL_TCGEN05_PAIR || p->residual)
            return fail(LEXB_ERR_UNSUPPORTED, "silu(gate) * up is fused into the two-CTA GEMM only (m > 8, n %% 128 == 0, k %% 256 == 0, no residual)");
        if (act && (rc = check_buf(act, g, m * (n / 2) * 2, "act"))) return rc;
    } else if (!gather && (rc = check_buf(y, g, m * n * 4, "y"))) return rc;
    if (gather && p->kernel != KERNEL_TCGEN05_PAIR)
        return fail(LEXB_ERR_UNSUPPORTED, "the fused all-gather exists in the two-CTA GEMM only (m > 16, n %% 128 == 0, k %% 256 == 0)");
    if (p->residual) {
        if ((rc = check_buf(r, g, m * n * 4, "r"))) return rc;
    } else if (r) {
        return fail(LEXB_ERR_ARG, "a residual buffer was bound to a pipeline planned without one");
    }
    if (p->kernel == KERNEL_TCGEN05 || p->kernel == KERNEL_TCGEN05_PAIR) {
        lexb_pipeline::MapEntry maps;
        if ((rc = get_maps(p, x->ptr, wq->ptr, ws->ptr, &maps))) return rc;
        lexb::GemmArgs a{};
        a.wq = static_cast<const uint8_t*>(wq->ptr);
        a.ws = static_cast<const uint8_t*>(ws->ptr);
        a.wg = static_cast<const float*>(wg->ptr);
        a.r = r ? static_cast<const float*>(r->ptr) : nullptr;
        a.y = y ? static_cast<float*>(y->ptr) : nullptr;
        a.act = act ? static_cast<uint16_t*>(act->ptr) : nullptr;
        a.silu_gather = (gather && gather->silu) ? 1u : 0u;
        lexb::GatherDst gd{};
        if (gather) {
            gd = *gather;
            for (uint32_t d = 0; d < gd.world; d++) a.gather_y[d] = gd.y[d];
            a.gather_world = gd.world; a.gather_n = gd.n_total; a.gather_n0 = gd.n0;
        }
        a.status = g->d_status;
        a.trace = (g->d_trace && p->kernel == KERNEL_TCGEN05_PAIR && p->grid <= g->trace_ctas) ? g->d_trace : nullptr;
        // with room for two launches the records alternate between the two halves, so that two launches in a row
        // can be read side by side (the gap between them on the GPU's global timer)
        if (a.trace && 2u * p->grid <= g->trace_ctas) a.trace += 16ull * p->grid * (g->trace_toggle++ & 1u);
        a.m = p->m; a.n = p->n; a.k = p->k;
        a.tm = p->tm; a.stages = p->stages; a.w_stages = p->w_stages; a.raw_stages = p->raw_stages; a.k_sub = p->k_sub; a.x_rows = p->x_rows;
        // bit 0: operand-collector hint; bit 1 (two-CTA kernel): the packed weights are constant - declared, or
        // proven from the step list - so their copy and decode may run ahead of the stream's order
        a.flags = p->flags | ((p->w_const || (order.early_weights && !p->w_volatile)) ? 2u : 0u);
        a.k_splits = p->k_splits; a.kb_per_split = p->kb_per_split; a.partial = p->partial; a.tok_blocks = p->tok_blocks;
        a.tmem_cols = p->tmem_cols; a.m_tiles = p->m_tiles; a.n_acc = p->n_acc;
        a.x_tx_bytes = p->kernel == KERNEL_TCGEN05_PAIR ? (p->m < p->x_rows ? p->m : p->x_rows) * 128u
                                                        : (p->tm < p->m ? p->tm : p->m) * 128u;
        if (p->kernel == KERNEL_TCGEN05_PAIR) {
            // Programmatic dependent launch: this kernel's blocks may be scheduled while the previous
            // launch of the stream drains (they wait for it before touching global memory), which
            // hides most of the gap between two launches.  LEXB_PDL=0 turns it off.
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3(p->grid);
            cfg.blockDim = dim3(p->threads);
            cfg.dynamicSmemBytes = p->smem;
            cfg.stream = g->stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = pdl ? 1 : 0;
            if (a.trace)
                LAUNCH_TRY(cudaLaunchKernelEx(&cfg, lexb::gemm_fp4_tcgen05_pair_kernel<true>, maps.map, maps.map_wq, maps.map_ws, a));
            else
                LAUNCH_TRY(cudaLaunchKernelEx(&cfg, lexb::gemm_fp4_tcgen05_pair_kernel<false>, maps.map, maps.map_wq, maps.map_ws, a));
            if (p->k_splits > 1) {
                CUDA_TRY(cudaGetLastError());
                const size_t elems = static_cast<size_t>(p->m) * p->n;       // n % 128 == 0: a multiple of 4
                const uint32_t blocks = static_cast<uint32_t>(std::min<size_t>((elems / 4 + 255) / 256, static_cast<size_t>(g->prop.multiProcessorCount) * 8u));
                cudaLaunchConfig_t rc_cfg{};
                rc_cfg.gridDim = dim3(blocks);
                rc_cfg.blockDim = dim3(256);
                rc_cfg.stream = g->stream;
                rc_cfg.attrs = attr;
                rc_cfg.numAttrs = g->pdl ? 1 : 0;
                LAUNCH_TRY(cudaLaunchKernelEx(&rc_cfg, lexb::splitk_reduce_kernel, static_cast<const float*>(p->partial), p->k_splits, elems,
                                            a.r, a.y, gd, a.act, p->n));
            }
        } else {
            INJECT_LAUNCH();
            lexb::gemm_fp4_tcgen05_kernel<<<p->grid, p->threads, p->smem, g->stream>>>(maps.map, a);
        }
    } else if (p->kernel == KERNEL_MATMUL_Q) {
        lexb_pipeline::MapEntry maps;
        if ((rc = get_maps(p, x->ptr, wq->ptr, ws->ptr, &maps))) return rc;
        lexb::MatmulQArgs a{};
        a.x = x->ptr;
        a.wg = static_cast<const float*>(wg->ptr);
        a.r = r ? static_cast<const float*>(r->ptr) : nullptr;
        a.y = static_cast<float*>(y->ptr);
        a.partial = p->partial;
        // the row tiles' arrival counters sit behind the partial products in the same allocation
        a.counters = p->partial ? reinterpret_cast<uint32_t*>(p->partial + static_cast<size_t>(p->k_splits) * p->m * p->n) : nullptr;
        a.status = g->d_status;
        a.m = p->m; a.n = p->n; a.k = p->k; a.stages = p->stages;
        a.k_splits = p->k_splits; a.kb_per_split = p->kb_per_split;
        a.ws_pitch = p->ws_pitch;
        a.flags = (p->w_const || (order.early_weights && !p->w_volatile)) ? 1u : 0u;
        lexb_pipeline::MapEntry nmaps = maps;         // placeholders when there is no hint (next_grid = 0)
        if (next && next->pipe && next->pipe->kernel == KERNEL_MATMUL_Q && next->pipe->gpu == g && next->wq && next->ws &&
            next->x && (a.flags & 1u) && get_maps(next->pipe, next->x->ptr, next->wq->ptr, next->ws->ptr, &nmaps) == LEXB_OK) {
            const lexb_pipeline* q = next->pipe;
            a.next_grid = q->grid; a.next_k_splits = q->k_splits; a.next_kb_per_split = q->kb_per_split;
            a.next_kb_all = q->k / lexb::MQ_STAGE_K; a.next_stages = q->stages; a.next_ws_pitch = q->ws_pitch;
        }
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(p->grid);
        cfg.blockDim = dim3(p->threads);
        cfg.dynamicSmemBytes = p->smem;
        cfg.stream = g->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = (g->pdl && (!order.fence || p->mq_pre)) ? 1 : 0;      // (behind the pieces kernel, that one is the fence)
        a.trace = (g->d_trace && p->grid <= g->trace_ctas) ? g->d_trace : nullptr;
        const size_t pieces_bytes = static_cast<size_t>(p->m) * 8u * (p->k / 2u), sfb_bytes = static_cast<size_t>(p->k / lexb::MQ_STAGE_K) * lexb::matmul_q_sfb_bytes(p->m);
        if (p->mq_pre) {
            a.pre_sfb = p->pre_buf + pieces_bytes;
            a.pre_amax = reinterpret_cast<const uint32_t*>(p->pre_buf + pieces_bytes + sfb_bytes);
            cudaLaunchConfig_t pc{};
            pc.gridDim = dim3(p->m, (p->k / lexb::MQ_STAGE_K + 31u) / 32u);      // a warp per stage
            pc.blockDim = dim3(1024);
            pc.stream = g->stream;
            pc.attrs = attr;
            pc.numAttrs = pdl ? 1 : 0;
            uint32_t* amax_w = reinterpret_cast<uint32_t*>(p->pre_buf + pieces_bytes + sfb_bytes);
            const float* no_xs = nullptr;
            if (p->x_q16) LAUNCH_TRY(cudaLaunchKernelEx(&pc, lexb::matmul_q_pieces_kernel<2>, static_cast<const void*>(x->ptr), p->k, p->pre_buf, p->pre_buf + pieces_bytes, amax_w, static_cast<const float*>(xs_q16->ptr)));
            else if (p->x_f32) LAUNCH_TRY(cudaLaunchKernelEx(&pc, lexb::matmul_q_pieces_kernel<1>, static_cast<const void*>(x->ptr), p->k, p->pre_buf, p->pre_buf + pieces_bytes, amax_w, no_xs));
            else LAUNCH_TRY(cudaLaunchKernelEx(&pc, lexb::matmul_q_pieces_kernel<0>, static_cast<const void*>(x->ptr), p->k, p->pre_buf, p->pre_buf + pieces_bytes, amax_w, no_xs));
        }
        const CUtensorMap& bmap = p->mq_pre ? p->pre_map : maps.map_wq;      // a placeholder without the pieces kernel
#define LEXB_MQ_LAUNCH(TR, XF, PR) LAUNCH_TRY(cudaLaunchKernelEx(&cfg, lexb::matmul_q_fp4_kernel<TR, XF, PR>, maps.map_wq, maps.map_ws, nmaps.map_wq, nmaps.map_ws, bmap, a))
        if (p->mq_pre) {
            if (p->x_f32) { if (a.trace) LEXB_MQ_LAUNCH(true, true, true); else LEXB_MQ_LAUNCH(false, true, true); }
            else { if (a.trace) LEXB_MQ_LAUNCH(true, false, true); else LEXB_MQ_LAUNCH(false, false, true); }
        } else {
            if (p->x_f32) { if (a.trace) LEXB_MQ_LAUNCH(true, true, false); else LEXB_MQ_LAUNCH(false, true, false); }
            else { if (a.trace) LEXB_MQ_LAUNCH(true, false, false); else LEXB_MQ_LAUNCH(false, false, false); }
        }
#undef LEXB_MQ_LAUNCH
    } else {
        lexb::MatvecArgs a{};
        a.x = static_cast<const __half*>(x->ptr);
        a.wq = static_cast<const uint8_t*>(wq->ptr);
        a.ws = static_cast<const uint8_t*>(ws->ptr);
        a.wg = static_cast<const float*>(wg->ptr);
        a.r = r ? static_cast<const float*>(r->ptr) : nullptr;
        a.y = static_cast<float*>(y->ptr);
        a.m = p->m; a.n = p->n; a.k = p->k; a.kc = p->kc;
        const bool ragged = (p->k % lexb::MV_SLICE) != 0u;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(p->grid);
        cfg.blockDim = dim3(p->threads);
        cfg.dynamicSmemBytes = p->smem;
        cfg.stream = g->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl ? 1 : 0;
        if (p->m > 8) {
            if (ragged) LAUNCH_TRY(cudaLaunchKernelEx(&cfg, lexb::matvec_fp4_kernel<true, true, false>, a));
            else LAUNCH_TRY(cudaLaunchKernelEx(&cfg, lexb::matvec_fp4_kernel<true, false, false>, a));
        } else if (lexb::matvec_uses_ring(p->m)) {
            if (ragged) LAUNCH_TRY(cudaLaunchKernelEx(&cfg, lexb::matvec_fp4_kernel<false, true, true>, a));
            else LAUNCH_TRY(cudaLaunchKernelEx(&cfg, lexb::matvec_fp4_kernel<false, false, true>, a));
        } else {
            if (ragged) LAUNCH_TRY(cudaLaunchKernelEx(&cfg, lexb::matvec_fp4_kernel<false, true, false>, a));
            else LAUNCH_TRY(cudaLaunchKernelEx(&cfg, lexb::matvec_fp4_kernel<false, false, false>, a));
        }
    }
    CUDA_TRY(cudaGetLastError());
    return LEXB_OK;
}

// Consecutive steps of a list that can run as one persistent kernel (matmul_q_chain_sm100.cuh): block-scaled
// matmul_q of up to 8 tokens with the default ring depth and digit-row source of their token count, one K range per block, the same
// t, k and activation type (n may differ), weights declared constant.  LEXB_CHAIN=0 turns it off.
// (two accumulator sets of 2 x 64 columns: 8 tokens x 8 digit rows)
static uint32_t chain_max_m() {
    static const uint32_t v = env_u32("LEXB_CHAIN_MAX_M", lexb::MQC_MAX_TOKENS);
    return v > lexb::MQC_MAX_TOKENS ? lexb::MQC_MAX_TOKENS : v;
}
// From this many tokens on the digit rows of a run come from matmul_q_pieces_kernel, not from piece warps in every block.
static uint32_t chain_pre_min_m() {
    static const uint32_t v = env_u32("LEXB_CHAIN_PRE_MIN_M", 3);
    return v;
}
// Address ranges a step reads and writes, for the dependence checks of a step list.
struct Range { const char *lo, *hi; };
inline bool meet(Range a, Range b) { return a.lo < b.hi && b.lo < a.hi; }
struct StepRanges {
    Range x{}, wq{}, ws{}, r{}, y{};
    bool valid = false;          // false: a null pipeline, buffer list or buffer (the step's own launch reports it)
};

StepRanges step_ranges(const lexb_step& s) {
    StepRanges out;
    const lexb_pipeline* p = s.pipeline;
    const uint32_t q = p && p->x_q16 ? 1u : 0u;       // int16 activations bring their scales as a second binding
    if (!p || !s.buffers || s.nbuffers != (p->residual ? 6u : 5u) + q) return out;
    for (uint32_t b = 0; b < s.nbuffers; b++)
        if (!s.buffers[b] || !s.buffers[b]->ptr) return out;
    auto range = [](const lexb_buffer* b, size_t bytes) { const char* p0 = static_cast<const char*>(b->ptr); return Range{p0, p0 + bytes}; };
    const size_t m = p->m, n = p->n, k = p->k, out_bytes = m * n * 4;
    out.x = range(s.buffers[0], m * k * (p->x_f32 ? 4 : 2));
    out.wq = range(s.buffers[1 + q], n * k / 2);
    out.ws = range(s.buffers[2 + q], n * k / 16);
    out.r = p->residual ? range(s.buffers[4 + q], out_bytes) : Range{nullptr, nullptr};
    out.y = range(s.buffers[(p->residual ? 5 : 4) + q], out_bytes);
    out.valid = true;
    return out;
}

// What the steps of one lexb_run_launches / lexb_time_launches call have written so far.  The call's first launch
// is a fence (it starts when all earlier work of the stream is done), so a later step whose packed weights meet
// none of these ranges reads weights that nothing in flight writes: its kernel may load them ahead of the
// stream's order.  That is proven here from the list, as the reference's in-order contract
// (crates/lex-cuda/src/device.rs:629-672) leaves no other way to know it.
struct ListProof {
    std::vector<Range> written;      // distinct y ranges
    bool weights_untouched(const StepRanges& s) const {
        for (const Range& w : written)
            if (meet(s.wq, w) || meet(s.ws, w)) return false;
        return true;
    }
    void add(const StepRanges& s) {
        for (const Range& w : written)
            if (w.lo == s.y.lo && w.hi == s.y.hi) return;
        written.push_back(s.y);
    }
};

bool chain_member(const lexb_gpu* g, const lexb_step& s, const lexb_pipeline* first) {
    const lexb_pipeline* p = s.pipeline;
    if (!p || !s.buffers || p->gpu != g || p->kernel != KERNEL_MATMUL_Q || p->x_q16 || p->m > chain_max_m() || p->k_splits != 1u) return false;
    if (p->mq_pre != (p->m > 4u)) return false;                                      // (a plan forced the other way by LEXB_MQ_PRE stays as planned)
    if (p->w_volatile || s.nbuffers != (p->residual ? 6u : 5u)) return false;
    if ((p->k / lexb::MQ_STAGE_K) % lexb::MQ_WS_GROUP == 1u) return false;          // a scale-byte group of one stage is seen by half the scale warps only
    if (p->stages != (p->m <= 4u ? lexb::MQ_MAX_STAGES : 7u) || lexb::matmul_q_chain_smem_bytes(p->stages, p->m) > g->smem_optin) return false;
    return !first || (p->m == first->m && p->k == first->k && p->x_f32 == first->x_f32 && p->stages == first->stages &&
                      p->ws_pitch == first->ws_pitch);
}

// Length of the run of steps starting at i that one persistent kernel can take (0: step i is launched on its own).
// The run's copy warp starts on the weights at once, so every member's weights must be declared constant or be
// untouched by the steps of this call so far (`proof`) and by the run's own members.
size_t chain_run(const lexb_gpu* g, const lexb_step* steps, size_t nsteps, size_t i, const ListProof& proof) {
    static const bool on = env_u32("LEXB_CHAIN", 1) != 0;
    if (!on || !chain_member(g, steps[i], nullptr)) return 0;
    const StepRanges first = step_ranges(steps[i]);
    if (!first.valid) return 0;                                  // a null buffer entry: the step's own launch reports it
    if (!steps[i].pipeline->w_const && !proof.weights_untouched(first)) return 0;
    // The run's row tiles are spread over the blocks with no order between blocks, so a step joins the run only
    // if nothing it reads (x, r, the weights) is written by a step already in it and nothing it writes (y) is
    // read or written by one: such a step starts the next launch, and the stream orders it.
    std::vector<StepRanges> in_run{first};
    auto conflicts = [&](const StepRanges& c, bool declared_const) {
        if (!declared_const && !proof.weights_untouched(c)) return true;
        for (const StepRanges& e : in_run) {
            if (meet(c.x, e.y) || meet(c.r, e.y) || meet(c.y, e.x) || meet(c.y, e.r) || meet(c.y, e.y)) return true;
            if (meet(c.wq, e.y) || meet(c.ws, e.y) || meet(c.y, e.wq) || meet(c.y, e.ws)) return true;
        }
        return false;
    };
    size_t len = 1;
    while (i + len < nsteps && len < 4096 && chain_member(g, steps[i + len], steps[i].pipeline)) {
        const StepRanges c = step_ranges(steps[i + len]);
        if (!c.valid || conflicts(c, steps[i + len].pipeline->w_const)) break;
        in_run.push_back(c);
        len++;
    }
    if (len >= 2) return len;
    // a single step with more row tiles than SMs: the persistent kernel takes them without a second wave of
    // block set-ups (n = 28672: 224 tiles)
    static const bool single = env_u32("LEXB_CHAIN_SINGLE", 1) != 0;
    const uint32_t tiles = (steps[i].pipeline->n + lexb::MQ_ROWS - 1u) / lexb::MQ_ROWS;
    return single && tiles > static_cast<uint32_t>(g->prop.multiProcessorCount) ? 1 : 0;
}

int launch_chain(lexb_gpu* g, const lexb_step* steps, size_t count, bool fence) {
    bool pdl_next = g->pdl && !fence;            // the run's first kernel launch is the fence, when one is asked for
    const lexb_pipeline* p0 = steps[0].pipeline;
    std::vector<lexb::MqChainJob> jobs(count);
    uint32_t tiles = 0, jobs_first_tiles = 0;        // (the latter: every step's tile count if they all agree, else 0)
    int rc;
    const bool pre = p0->m >= chain_pre_min_m() || p0->m > 4u;       // (the piece warps of a block take up to 4 tokens)
    std::vector<const void*> pre_done;               // activation buffers whose digit rows this run has asked for
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    const size_t pieces_bytes = static_cast<size_t>(p0->m) * 8u * (p0->k / 2u);
    const size_t sfb_bytes = static_cast<size_t>(p0->k / lexb::MQ_STAGE_K) * lexb::MQ_SF_BYTES;
    for (size_t i = 0; i < count; i++) {
        const lexb_pipeline* p = steps[i].pipeline;
        lexb_buffer* const* b = steps[i].buffers;
        const lexb_buffer *x = b[0], *wq = b[1], *ws = b[2], *wg = b[3], *r = p->residual ? b[4] : nullptr;
        const lexb_buffer* y = p->residual ? b[5] : b[4];
        const size_t m = p->m, n = p->n, k = p->k;
        if ((rc = check_buf(x, g, m * k * (p->x_f32 ? 4 : 2), "x"))) return rc;
        if ((rc = check_buf(wq, g, n * k / 2, "wq"))) return rc;
        if ((rc = check_buf(ws, g, n * k / 16, "ws"))) return rc;
        if ((rc = check_buf(wg, g, n * 4, "wg"))) return rc;
        if ((rc = check_buf(y, g, m * n * 4, "y"))) return rc;
        if (r && (rc = check_buf(r, g, m * n * 4, "r"))) return rc;
        lexb_pipeline::MapEntry maps;
        if ((rc = get_maps(p, x->ptr, wq->ptr, ws->ptr, &maps))) return rc;
        jobs[i].wq = maps.map_wq;
        jobs[i].ws = maps.map_ws;
        jobs[i].x = x->ptr;
        jobs[i].wg = static_cast<const float*>(wg->ptr);
        jobs[i].r = r ? static_cast<const float*>(r->ptr) : nullptr;
        jobs[i].y = static_cast<float*>(y->ptr);
        jobs[i].n = p->n;
        if (pre) {
            const auto key = std::make_tuple(static_cast<const void*>(x->ptr), p0->m, p0->k, p0->x_f32 != 0, g->stream);
            auto it = g->chain_pre.find(key);
            if (it == g->chain_pre.end()) {
                if (g->chain_pre.size() >= 256 && pre_done.empty()) {
                    // activation buffers come and go: start over (buffers of launches in flight are freed after them;
                    // not in the middle of a run, whose earlier jobs point into these buffers)
                    CUDA_TRY(cudaDeviceSynchronize());
                    for (auto& e : g->chain_pre) cudaFree(e.second.buf);
                    g->chain_pre.clear();
                }
                lexb_gpu::ChainPre cp{};
                const size_t total = pieces_bytes + sfb_bytes + 4u * lexb::MQ_MAX_TOKENS;
                CUDA_TRY(x_malloc(&cp.buf, total));
                cudaError_t e = cudaMemsetAsync(cp.buf, 0, total, g->stream);      // scale rows nobody writes stay zero
                int erc = e == cudaSuccess ? encode_2d(p, &cp.map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, cp.buf, p0->k / 2u, 8u * p0->m, 128u,
                                                      8u * p0->m, CU_TENSOR_MAP_SWIZZLE_128B, "digit rows of a run")
                                           : fail(LEXB_ERR_CUDA, "clearing the digit-row buffers: %s", cudaGetErrorString(e));
                if (erc) { cudaFree(cp.buf); return erc; }
                it = g->chain_pre.emplace(key, cp).first;
            }
            uint8_t* buf = it->second.buf;
            jobs[i].pre = it->second.map;
            jobs[i].pre_sfb = buf + pieces_bytes;
            jobs[i].pre_amax = reinterpret_cast<const uint32_t*>(buf + pieces_bytes + sfb_bytes);
            if (std::find(pre_done.begin(), pre_done.end(), x->ptr) == pre_done.end()) {
                pre_done.push_back(x->ptr);
                cudaLaunchConfig_t pc{};
                pc.gridDim = dim3(p0->m, (p0->k / lexb::MQ_STAGE_K + 31u) / 32u);      // a warp per stage
                pc.blockDim = dim3(1024);
                pc.stream = g->stream;
                pc.attrs = attr;
                pc.numAttrs = pdl_next ? 1 : 0;
                pdl_next = g->pdl;
                uint32_t* amax_w = reinterpret_cast<uint32_t*>(buf + pieces_bytes + sfb_bytes);
                const float* no_xs = nullptr;
                if (p0->x_f32) LAUNCH_TRY(cudaLaunchKernelEx(&pc, lexb::matmul_q_pieces_kernel<1>, static_cast<const void*>(x->ptr), p0->k, buf, buf + pieces_bytes, amax_w, no_xs));
                else LAUNCH_TRY(cudaLaunchKernelEx(&pc, lexb::matmul_q_pieces_kernel<0>, static_cast<const void*>(x->ptr), p0->k, buf, buf + pieces_bytes, amax_w, no_xs));
            }
        }
        const uint32_t job_tiles = (p->n + lexb::MQ_ROWS - 1u) / lexb::MQ_ROWS;
        if (i == 0) jobs_first_tiles = job_tiles;
        else if (job_tiles != jobs_first_tiles) jobs_first_tiles = 0;
        tiles += job_tiles;
        jobs[i].tile_end = tiles;
    }
    const size_t table_bytes = sizeof(lexb::MqChainJob) * count;
    uint64_t h = 1469598103934665603ull;
    {
        const unsigned char* bytes = reinterpret_cast<const unsigned char*>(jobs.data());
        for (size_t i = 0; i < table_bytes; i++) h = (h ^ bytes[i]) * 1099511628211ull;
    }
    lexb::MqChainJob* d_jobs = nullptr;
    auto hit = g->chain_tables.equal_range(h);
    for (auto it = hit.first; it != hit.second && !d_jobs; ++it)
        if (it->second.host.size() == count && !memcmp(it->second.host.data(), jobs.data(), table_bytes)) d_jobs = it->second.dev;
    if (!d_jobs) {
        if (g->chain_tables.size() >= 4096) {
            // (tables of launches still in flight are freed only after them)
            CUDA_TRY(cudaStreamSynchronize(g->stream));
            for (auto& e : g->chain_tables) cudaFree(e.second.dev);
            g->chain_tables.clear();
        }
        CUDA_TRY(x_malloc(&d_jobs, table_bytes));
        auto it = g->chain_tables.emplace(h, lexb_gpu::ChainTable{std::move(jobs), d_jobs});
        // (the source is the cache's own copy: it outlives the transfer)
        CUDA_TRY_AT(SITE_COPY, cudaMemcpyAsync(d_jobs, it->second.host.data(), table_bytes, cudaMemcpyHostToDevice, g->stream));
    }
    lexb::MqChainArgs a{};
    a.jobs = d_jobs;
    a.n_jobs = static_cast<uint32_t>(count);
    a.n_tiles = tiles;
    a.tiles_per_job = jobs_first_tiles;
    a.m = p0->m; a.k = p0->k; a.stages = p0->stages; a.ws_pitch = p0->ws_pitch;
    a.status = g->d_status;
    // blocks of this kernel do not wait for one another, and there is at most one per SM
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(std::min<uint32_t>(tiles, static_cast<uint32_t>(g->prop.multiProcessorCount)));
    cfg.blockDim = dim3(pre ? lexb::MQC_THREADS_PRE : lexb::MQC_THREADS);
    cfg.dynamicSmemBytes = lexb::matmul_q_chain_smem_bytes(p0->stages, p0->m);
    cfg.stream = g->stream;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_next ? 1 : 0;
    if (pre) {
        if (p0->x_f32) LAUNCH_TRY(cudaLaunchKernelEx(&cfg, lexb::matmul_q_chain_kernel<true, true>, a));
        else LAUNCH_TRY(cudaLaunchKernelEx(&cfg, lexb::matmul_q_chain_kernel<false, true>, a));
    } else {
        if (p0->x_f32) LAUNCH_TRY(cudaLaunchKernelEx(&cfg, lexb::matmul_q_chain_kernel<true, false>, a));
        else LAUNCH_TRY(cudaLaunchKernelEx(&cfg, lexb::matmul_q_chain_kernel<false, false>, a));
    }
    return LEXB_OK;
}

int launch_step(lexb_gpu* g, const lexb_step& s, const lexb_step* following = nullptr, Order order = Order{}) {
    if (!s.pipeline || !s.buffers) return fail(LEXB_ERR_ARG, "step without pipeline or buffers");
    const bool res = s.pipeline->residual;
    const uint32_t q = s.pipeline->x_q16 ? 1u : 0u;
    if (s.nbuffers != (res ? 6u : 5u) + q)
        return fail(LEXB_ERR_ARG, "step binds %u buffers, the pipeline takes %u: [%s, wq, ws, wg, %sy]", s.nbuffers,
                    (res ? 6u : 5u) + q, q ? "xq, xs" : "x", res ? "r, " : "");
    if (q) {
        // matmul_int8's bindings (crates/lex-msl/src/int8.rs:121-125): [xq, xs, wq, ws, wg, (r), y]
        lexb_buffer* const* c = s.buffers;
        return launch_one(g, s.pipeline, c[0], c[2], c[3], c[4], res ? c[5] : nullptr, res ? c[6] : c[5], nullptr, nullptr, order,
                          nullptr, c[1]);
    }
    lexb_buffer* const* b = s.buffers;
    NextWeights nw{};
    static const bool hints = env_u32("LEXB_NEXT_HINT", 1) != 0;     // LEXB_NEXT_HINT=0: no prefetch of the next step's weights
    if (hints && following && following->pipeline && following->buffers && following->nbuffers >= 5u && !following->pipeline->x_q16)
        nw = NextWeights{following->pipeline, following->buffers[0], following->buffers[1], following->buffers[2]};
    return launch_one(g, s.pipeline, b[0], b[1], b[2], b[3], res ? b[4] : nullptr, res ? b[5] : b[4], nullptr,
                      nw.pipe ? &nw : nullptr, order);
}

// Issues the steps of a list once, in order, forming runs; `proof` and `first` carry over between the passes of
// lexb_time_launches.  `first`: nothing of this call has been launched yet - that launch is the call's fence.
int issue_list(lexb_gpu* g, const lexb_step* steps, size_t nsteps, ListProof& proof, bool& first, const lexb_step* after_last) {
    int rc;
    for (size_t i = 0; i < nsteps;) {
        if (const size_t len = chain_run(g, steps, nsteps, i, proof)) {
            if ((rc = launch_chain(g, steps + i, len, first))) return rc;
            for (size_t e = i; e < i + len; e++) proof.add(step_ranges(steps[e]));
            first = false;
            i += len;
            continue;
        }
        const StepRanges sr = step_ranges(steps[i]);
        Order order;
        order.fence = first;
        order.early_weights = sr.valid && proof.weights_untouched(sr);
        const lexb_step* following = i + 1 < nsteps ? &steps[i + 1] : after_last;
        if ((rc = launch_step(g, steps[i], following, order))) return rc;
        if (sr.valid) proof.add(sr);
        first = false;
        i++;
    }
    return LEXB_OK;
}

}  // namespace

extern "C" {

const char* lexb_last_error(void) { return g_last_error.c_str(); }
const char* lexb_version(void) { return "lexb 0.1 (sm_100a; gemm_fp4: tcgen05 GEMM + split-K matvec)"; }

int lexb_open(int device, lexb_gpu** out) {
    if (!out) return fail(LEXB_ERR_ARG, "lexb_open: null out");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(LEXB_ERR_UNSUPPORTED, "no CUDA device (%s); this library has no CPU path", cudaGetErrorString(e));
    if (device < 0 || device >= count) return fail(LEXB_ERR_ARG, "device %d out of range (%d devices)", device, count);
    lexb_gpu* g = new (std::nothrow) lexb_gpu();
    if (!g) return fail(LEXB_ERR_ARG, "out of host memory");
    g->device = device;
    auto bail = [&](int code) { lexb_close(g); return code; };
    if (cudaSetDevice(device) != cudaSuccess) return bail(fail(LEXB_ERR_CUDA, "cudaSetDevice(%d) failed", device));
    if (cudaGetDeviceProperties(&g->prop, device) != cudaSuccess) return bail(fail(LEXB_ERR_CUDA, "cudaGetDeviceProperties failed"));
    if (g->prop.major != 10)
        return bail(fail(LEXB_ERR_UNSUPPORTED, "device %d is %s (compute %d.%d); the kernels are built for sm_100a only",
                         device, g->prop.name, g->prop.major, g->prop.minor));
    g->smem_optin = g->prop.sharedMemPerBlockOptin;
    g->pdl = env_u32("LEXB_PDL", 1) != 0;
    if (cudaStreamCreateWithFlags(&g->own_stream, cudaStreamNonBlocking) != cudaSuccess)
        return bail(fail(LEXB_ERR_CUDA, "cudaStreamCreate failed"));
    g->stream = g->own_stream;
    if (cudaMalloc(&g->d_status, sizeof(uint32_t)) != cudaSuccess || cudaMemsetAsync(g->d_status, 0, sizeof(uint32_t), g->stream) != cudaSuccess ||
        cudaStreamSynchronize(g->stream) != cudaSuccess)
        return bail(fail(LEXB_ERR_CUDA, "allocating the status word failed"));
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn ||
        qres != cudaDriverEntryPointSuccess)
        return bail(fail(LEXB_ERR_CUDA, "the driver does not export cuTensorMapEncodeTiled"));
    g->encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    const int max_smem = static_cast<int>(g->smem_optin);
    if (cudaFuncSetAttribute(lexb::gemm_fp4_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::gemm_fp4_tcgen05_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::gemm_fp4_tcgen05_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matvec_fp4_kernel<true, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matvec_fp4_kernel<true, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matvec_fp4_kernel<false, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matvec_fp4_kernel<false, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matvec_fp4_kernel<false, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matvec_fp4_kernel<false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matmul_q_chain_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matmul_q_chain_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matmul_q_chain_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matmul_q_chain_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matmul_q_fp4_kernel<true, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matmul_q_fp4_kernel<false, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matmul_q_fp4_kernel<true, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matmul_q_fp4_kernel<false, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matmul_q_fp4_kernel<true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matmul_q_fp4_kernel<false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matmul_q_fp4_kernel<true, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess ||
        cudaFuncSetAttribute(lexb::matmul_q_fp4_kernel<false, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem) != cudaSuccess)
        return bail(fail(LEXB_ERR_CUDA, "cudaFuncSetAttribute(max dynamic shared memory) failed: %s", cudaGetErrorString(cudaGetLastError())));
    *out = g;
    return LEXB_OK;
}

void lexb_close(lexb_gpu* g) {
    if (!g) return;
    cudaSetDevice(g->device);
    if (g->own_stream) {
        cudaStreamSynchronize(g->own_stream);
        cudaStreamDestroy(g->own_stream);
    }
    if (g->d_status) cudaFree(g->d_status);
    if (g->d_trace) cudaFree(g->d_trace);
    for (auto& e : g->chain_tables) cudaFree(e.second.dev);
    g->chain_tables.clear();
    for (auto& e : g->chain_pre) cudaFree(e.second.buf);
    g->chain_pre.clear();
    delete g;
}

int lexb_info(lexb_gpu* g, lexb_device_info* out) {
    int rc = use(g);
    if (rc) return rc;
    if (!out) return fail(LEXB_ERR_ARG, "lexb_info: null out");
    memset(out, 0, sizeof *out);
    snprintf(out->name, sizeof out->name, "%s", g->prop.name);
    out->cc_major = g->prop.major;
    out->cc_minor = g->prop.minor;
    out->sm_count = g->prop.multiProcessorCount;
    out->unified_memory = 0;
    out->max_threadgroup_bytes = g->smem_optin;
    out->recommended_working_set_bytes = g->prop.totalGlobalMem;
    out->l2_bytes = static_cast<size_t>(g->prop.l2CacheSize);
    return LEXB_OK;
}

int lexb_set_stream(lexb_gpu* g, void* cuda_stream) {
    int rc = use(g);
    if (rc) return rc;
    g->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : g->own_stream;
    return LEXB_OK;
}
void* lexb_get_stream(lexb_gpu* g) { return g ? static_cast<void*>(g->stream) : nullptr; }

int lexb_sync(lexb_gpu* g) {
    int rc = use(g);
    if (rc) return rc;
    CUDA_TRY(cudaStreamSynchronize(g->stream));
    return LEXB_OK;
}

int lexb_alloc(lexb_gpu* g, size_t bytes, lexb_buffer** out) {
    int rc = use(g);
    if (rc) return rc;
    if (!out) return fail(LEXB_ERR_ARG, "lexb_alloc: null out");
    *out = nullptr;
    void* p = nullptr;
    CUDA_TRY(x_malloc(&p, bytes ? bytes : 1));
    lexb_buffer* b = new (std::nothrow) lexb_buffer{g, p, bytes, true};
    if (!b) {
        cudaFree(p);
        return fail(LEXB_ERR_ARG, "out of host memory");
    }
    *out = b;
    return LEXB_OK;
}

int lexb_zeroed(lexb_gpu* g, size_t bytes, lexb_buffer** out) {
    int rc = lexb_alloc(g, bytes, out);
    if (rc) return rc;
    if (bytes) {
        cudaError_t e = cudaMemsetAsync((*out)->ptr, 0, bytes, g->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(g->stream);
        if (e != cudaSuccess) {
            lexb_free(*out);
            *out = nullptr;
            return fail(LEXB_ERR_CUDA, "zeroing %zu bytes failed: %s", bytes, cudaGetErrorString(e));
        }
    }
    return LEXB_OK;
}

int lexb_wrap(lexb_gpu* g, void* device_ptr, size_t bytes, lexb_buffer** out) {
    if (!g || !out) return fail(LEXB_ERR_ARG, "lexb_wrap: null argument");
    if (!device_ptr && bytes) return fail(LEXB_ERR_ARG, "lexb_wrap: null device pointer");
    lexb_buffer* b = new (std::nothrow) lexb_buffer{g, device_ptr, bytes, false};
    if (!b) return fail(LEXB_ERR_ARG, "out of host memory");
    *out = b;
    return LEXB_OK;
}

int lexb_free(lexb_buffer* b) {
    if (!b) return LEXB_OK;
    int rc = LEXB_OK;
    if (b->owned && b->ptr) {
        cudaSetDevice(b->gpu->device);
        cudaError_t e = cudaFree(b->ptr);
        if (e != cudaSuccess) rc = fail(LEXB_ERR_CUDA, "cudaFree: %s", cudaGetErrorString(e));
    }
    delete b;
    return rc;
}

void* lexb_buffer_ptr(const lexb_buffer* b) { return b ? b->ptr : nullptr; }
size_t lexb_buffer_bytes(const lexb_buffer* b) { return b ? b->bytes : 0; }

int lexb_upload(lexb_gpu* g, lexb_buffer* dst, size_t off, const void* src, size_t bytes) {
    int rc = use(g);
    if (rc) return rc;
    if (!dst || (!src && bytes)) return fail(LEXB_ERR_ARG, "lexb_upload: null argument");
    if (off > dst->bytes || bytes > dst->bytes - off)
        return fail(LEXB_ERR_ARG, "lexb_upload: %zu bytes at offset %zu overrun a buffer of %zu", bytes, off, dst->bytes);
    CUDA_TRY_AT(SITE_COPY, cudaMemcpyAsync(static_cast<char*>(dst->ptr) + off, src, bytes, cudaMemcpyHostToDevice, g->stream));
    CUDA_TRY(cudaStreamSynchronize(g->stream));
    return LEXB_OK;
}

int lexb_download(lexb_gpu* g, const lexb_buffer* src, size_t off, void* dst, size_t bytes) {
    int rc = use(g);
    if (rc) return rc;
    if (!src || (!dst && bytes)) return fail(LEXB_ERR_ARG, "lexb_download: null argument");
    if (off > src->bytes || bytes > src->bytes - off)
        return fail(LEXB_ERR_ARG, "lexb_download: %zu bytes at offset %zu overrun a buffer of %zu", bytes, off, src->bytes);
    CUDA_TRY_AT(SITE_COPY, cudaMemcpyAsync(dst, static_cast<const char*>(src->ptr) + off, bytes, cudaMemcpyDeviceToHost, g->stream));
    CUDA_TRY(cudaStreamSynchronize(g->stream));
    return LEXB_OK;
}

int lexb_memset(lexb_gpu* g, lexb_buffer* dst, int byte, size_t bytes) {
    int rc = use(g);
    if (rc) return rc;
    if (!dst) return fail(LEXB_ERR_ARG, "lexb_memset: null buffer");
    if (bytes > dst->bytes) return fail(LEXB_ERR_ARG, "lexb_memset: %zu bytes overrun a buffer of %zu", bytes, dst->bytes);
    CUDA_TRY(cudaMemsetAsync(dst->ptr, byte, bytes, g->stream));
    return LEXB_OK;
}

int lexb_host_alloc(size_t bytes, void** out) {
    if (!out) return fail(LEXB_ERR_ARG, "lexb_host_alloc: null out");
    CUDA_TRY(cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault));
    return LEXB_OK;
}
int lexb_host_free(void* p) {
    if (p) CUDA_TRY(cudaFreeHost(p));
    return LEXB_OK;
}

int lexb_gemm_fp4_plan(lexb_gpu* g, uint32_t m, uint32_t n, uint32_t k, int residual, const lexb_sched* sched,
                       lexb_pipeline** out) {
    int rc = use(g);
    if (rc) return rc;
    if (!out) return fail(LEXB_ERR_ARG, "lexb_gemm_fp4_plan: null out");
    *out = nullptr;
    if (m == 0 || n == 0 || k == 0) return fail(LEXB_ERR_SHAPE, "gemm_fp4: empty extent (m=%u n=%u k=%u)", m, n, k);
    lexb_sched s{};
    if (sched) s = *sched;
    if (!s.kernel) s.kernel = env_u32("LEXB_KERNEL", 0);
    if (!s.tm) s.tm = env_u32("LEXB_TM", 0);
    if (!s.stages) s.stages = env_u32("LEXB_STAGES", 0);
    if (!s.kc) s.kc = env_u32("LEXB_KC", 0);
    if (!s.w_stages) s.w_stages = env_u32("LEXB_WSTAGES", 0);
    if (!s.k_splits) s.k_splits = env_u32("LEXB_KSPLITS", 0);
    // m <= 8: matvec (it also takes 9..16 when asked, but the GEMMs are faster there).  Otherwise the
    // two-CTA GEMM when the shape allows it (k in blocks of 256); the one-CTA kernel takes the rest.
    uint32_t kernel = s.kernel;
    if (!kernel) {
        if (m <= 8 || ((n % lexb::GEMM_TN || k % lexb::GEMM_BK) && m <= 16)) kernel = KERNEL_MATVEC;
        else if (n % lexb::GEMM_TN == 0 && k % lexb::PAIR_RAW_K == 0)
            kernel = KERNEL_TCGEN05_PAIR;
        else kernel = KERNEL_TCGEN05;
    }
    if (kernel == KERNEL_MATVEC && m > 16) return fail(LEXB_ERR_SHAPE, "the matvec kernel takes m <= 16, not %u", m);
    if (kernel < KERNEL_MATVEC || kernel > KERNEL_MATMUL_Q) return fail(LEXB_ERR_ARG, "unknown kernel selector %u", kernel);

    lexb_pipeline* p = new (std::nothrow) lexb_pipeline();
    if (!p) return fail(LEXB_ERR_ARG, "out of host memory");
    p->gpu = g;
    p->kernel = kernel;
    p->m = m; p->n = n; p->k = k;
    p->residual = residual != 0;
    auto bail = [&](int code) { lexb_pipeline_free(p); return code; };
    const char* stem = residual ? "gemm_fp4_res" : "gemm_fp4";
    p->w_const = (s.flags & LEXB_SCHED_WEIGHTS_CONSTANT) != 0u;
    p->w_volatile = (s.flags & LEXB_SCHED_WEIGHTS_MAY_CHANGE) != 0u;
    if (p->w_const && p->w_volatile)
        return bail(fail(LEXB_ERR_ARG, "LEXB_SCHED_WEIGHTS_CONSTANT and LEXB_SCHED_WEIGHTS_MAY_CHANGE exclude one another"));

    if (kernel == KERNEL_MATMUL_Q) {
        // Only through lexb_matmul_fp4_plan or an explicit selector: its arithmetic is matmul_q_x's
        // (weights not rounded to f16), within gemm_fp4's tolerance but not its rounding.
        if (m > lexb::MQ_MAX_TOKENS) return bail(fail(LEXB_ERR_SHAPE, "the block-scaled kernel takes at most %u tokens, not %u", lexb::MQ_MAX_TOKENS, m));
        if (n % lexb::MQ_ROWS) return bail(fail(LEXB_ERR_SHAPE, "matmul_q (nvfp4): %u rows per block do not divide n = %u", lexb::MQ_ROWS, n));
        if (k % lexb::MQ_STAGE_K) return bail(fail(LEXB_ERR_SHAPE, "matmul_q (nvfp4): blocks of %u columns do not divide k = %u", lexb::MQ_STAGE_K, k));
        uint32_t stages = s.stages ? s.stages : (m <= 4u ? lexb::MQ_MAX_STAGES : (m <= 8u ? 7u : (m <= 16u ? 5u : 3u)));     // what fits shared memory
        const uint32_t max_stages = m <= 16u ? lexb::MQ_MAX_STAGES : lexb::MQ_WIDE_MAX_STAGES;    // ... and, past 16 tokens, tensor memory
        if (stages < 2 || stages > max_stages || lexb::matmul_q_smem_bytes(m, stages) > g->smem_optin)
            return bail(fail(LEXB_ERR_ARG, "stages = %u outside [2, %u] or over the shared-memory limit", stages, max_stages));
        const uint32_t tiles = n / lexb::MQ_ROWS, kb_all = k / lexb::MQ_STAGE_K;
        const uint32_t sms = static_cast<uint32_t>(g->prop.multiProcessorCount);
        // one K range per block; split K when the row tiles alone leave most SMs idle
        uint32_t splits = s.k_splits ? s.k_splits : (tiles * 2u <= sms ? sms / tiles : 1u);
        if (splits > 8u) splits = 8u;
        while (splits > 1u && kb_all / splits < 4u) splits--;
        if (splits < 1u) splits = 1u;
        const uint32_t per = (kb_all + splits - 1u) / splits;
        splits = (kb_all + per - 1u) / per;
        p->k_splits = splits; p->kb_per_split = per; p->stages = stages;
        p->ws_pitch = k / 16u < 16u * lexb::MQ_WS_GROUP ? k / 16u : 16u * lexb::MQ_WS_GROUP;
        // In order by default, as the reference's launches are (crates/lex-cuda/src/device.rs:629-672): wq/ws are
        // loaded ahead of the stream's order only when the caller declares them constant or a step list shows
        // that nothing in flight writes them (ListProof); never when the caller says they may change.
        p->flags = 0u;
        if (splits > 1u) {
            // partial products [splits][m][n], then one arrival counter per row tile (zero between launches)
            const size_t pbytes = sizeof(float) * splits * static_cast<size_t>(m) * n;
            cudaError_t e = x_malloc(&p->partial, pbytes + sizeof(uint32_t) * tiles);
            // cleared on the launch stream and waited for: a launch on any stream may follow at once
            if (e == cudaSuccess) e = cudaMemsetAsync(reinterpret_cast<char*>(p->partial) + pbytes, 0, sizeof(uint32_t) * tiles, g->stream);
            if (e == cudaSuccess) e = cudaStreamSynchronize(g->stream);
            if (e != cudaSuccess) return bail(fail(LEXB_ERR_CUDA, "allocating the split-K workspace: %s", cudaGetErrorString(e)));
        }
        // From 5 tokens on the digit rows are derived once per launch by a small kernel ahead of this one
        // (each block deriving them itself is what bounds the kernel there); LEXB_MQ_PRE=0/1 forces either way.
        // (past 16 tokens there is no in-block path; int16 activations are widened by the pieces kernel only)
        p->x_q16 = t_plan_q16;
        p->mq_pre = m > 16u || p->x_q16 || env_u32("LEXB_MQ_PRE", m > 4u ? 1u : 0u) != 0;
        if (p->mq_pre) {
            const size_t pieces_bytes = static_cast<size_t>(m) * 8u * (k / 2u), sfb_bytes = static_cast<size_t>(kb_all) * lexb::matmul_q_sfb_bytes(m);
            const size_t total = pieces_bytes + sfb_bytes + 4u * lexb::MQ_MAX_TOKENS;
            cudaError_t e = x_malloc(&p->pre_buf, total);
            if (e == cudaSuccess) e = cudaMemsetAsync(p->pre_buf, 0, total, g->stream);          // scale rows nobody writes stay zero
            if (e == cudaSuccess) e = cudaStreamSynchronize(g->stream);
            if (e != cudaSuccess) return bail(fail(LEXB_ERR_CUDA, "allocating the digit-row buffers: %s", cudaGetErrorString(e)));
            int erc = encode_2d(p, &p->pre_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p->pre_buf, k / 2u, 8u * m, 128u, 8u * m,
                                CU_TENSOR_MAP_SWIZZLE_128B, "digit rows");
            if (erc) return bail(erc);
        }
        p->grid = tiles * splits;
        p->threads = p->mq_pre ? 32u * (2u + lexb::MQ_SCALE_WARPS) : lexb::MQ_THREADS;
        p->smem = lexb::matmul_q_smem_bytes(m, stages);
        p->tm = m;
        if (p->entry[0] == 0)
            snprintf(p->entry, sizeof p->entry, "%s_%u_%u_%u_%u_%u_%u", stem, m, n, k, m, lexb::MQ_ROWS, lexb::MQ_STAGE_K);
    } else if (kernel == KERNEL_TCGEN05) {
        if (n % lexb::GEMM_TN) return bail(fail(LEXB_ERR_SHAPE, "gemm_fp4: bn = %u does not divide n = %u", lexb::GEMM_TN, n));
        if (k % lexb::GEMM_BK) return bail(fail(LEXB_ERR_SHAPE, "gemm_fp4: bk = %u does not divide k = %u", lexb::GEMM_BK, k));
        uint32_t tm = s.tm;
        if (!tm) {
            const uint32_t tiles = (m + 255u) / 256u;
            tm = round_up((m + tiles - 1u) / tiles, 16u);
        }
        if (tm < 16 || tm > 256 || tm % 16) return bail(fail(LEXB_ERR_ARG, "tm = %u is not a multiple of 16 in [16, 256]", tm));
        const uint32_t stage_bytes = lexb::gemm_stage_bytes(tm);
        uint32_t max_stages = 0;
        while (max_stages < 12 && lexb::gemm_smem_bytes(tm, max_stages + 1) <= g->smem_optin) max_stages++;
        if (max_stages < 2) return bail(fail(LEXB_ERR_UNSUPPORTED, "tm = %u leaves room for %u stages (%u bytes each)", tm, max_stages, stage_bytes));
        uint32_t stages = s.stages ? s.stages : max_stages;
        if (stages < 2 || stages > max_stages) return bail(fail(LEXB_ERR_ARG, "stages = %u outside [2, %u] for tm = %u", stages, max_stages, tm));
        // two alternating accumulators whenever they fit the 512 columns of TMEM
        const uint32_t n_acc = 2;
        uint32_t cols = 32;
        while (cols < n_acc * tm) cols *= 2;
        p->tm = tm; p->stages = stages; p->tmem_cols = cols; p->n_acc = n_acc; p->m_tiles = (m + tm - 1) / tm;
        p->grid = p->m_tiles * (n / lexb::GEMM_TN);
        p->threads = lexb::GEMM_THREADS;
        p->smem = lexb::gemm_smem_bytes(tm, stages);
        snprintf(p->entry, sizeof p->entry, "%s_%u_%u_%u_%u_%u_%u", stem, m, n, k, tm, lexb::GEMM_TN, lexb::GEMM_BK);
    } else if (kernel == KERNEL_TCGEN05_PAIR) {
        if (n % lexb::GEMM_TN) return bail(fail(LEXB_ERR_SHAPE, "gemm_fp4 (pair): %u rows per CTA do not divide n = %u", lexb::GEMM_TN, n));
        if (k % lexb::PAIR_RAW_K) return bail(fail(LEXB_ERR_SHAPE, "gemm_fp4 (pair): the packed-weight block of %u columns does not divide k = %u", lexb::PAIR_RAW_K, k));
        // Tiles of 512 tokens (two blocks of 256: each weight decoded once for 512 tokens), 256, 128 or 64 (one block;
        // the MMAs' N shrinks with it, the decode per tile does not); tm asks for one of them at any m
        if (s.tm && s.tm != 64u && s.tm != 128u && s.tm != 256u && s.tm != 512u)
            return bail(fail(LEXB_ERR_ARG, "tm = %u: the two-CTA kernel's tiles hold 64, 128, 256 or 512 tokens", s.tm));
        p->tm = s.tm ? s.tm : (m > 256u ? 512u : m > 128u ? 256u : m > 64u ? 128u : 64u);
        p->tok_blocks = p->tm == 512u ? 2u : 1u;
        p->flags = env_u32("LEXB_COLLECTOR", 0) ? 1u : 0u; p->tmem_cols = lexb::PAIR_TMEM_COLS; p->n_acc = 1;
        p->m_tiles = (m + p->tm - 1) / p->tm;
        const uint32_t n_pairs = (n + 2u * lexb::GEMM_TN - 1) / (2u * lexb::GEMM_TN);
        // Two ways to fill the SM pairs when whole tiles fill them badly (few tiles, or a short last wave).  Split K:
        // each split takes whole blocks of 256 columns (at least 4) and writes a partial product that a second
        // launch sums.  Smaller tiles: more of them; every weight is decoded once per tile of tokens, but a tile's
        // partial product and its store shrink with it and fewer splits are needed.  (Below 256 tokens a K step
        // costs the same: it is the decode that bounds it, not the MMAs.)
        // Every (tile, splits) pair is priced with figures fitted to 159 launches timed on a B200 (us; rms error
        // 4 %): 4.5 overall; per wave of tiles 8.05 / 5.3 / 4.0 / 4.1 for a block's start and its store of a
        // 512 / 256 / 128 / 64-token tile and 0.559 / 0.311 / 0.310 / 0.304 per K step; for the reduction launch its
        // bytes at 3.33 TB/s minus 1.1.  The cheapest wins; a smaller tile or a further split must win by 2 %.
        const uint32_t sm_pairs = static_cast<uint32_t>(g->prop.multiProcessorCount) / 2u;
        const uint32_t raw_blocks = k / lexb::PAIR_RAW_K;
        uint32_t splits = s.k_splits ? s.k_splits : 1u;
        {
            // per tile size 512 / 256 / 128 / 64: us per K step, us per wave for a block's start and store
            static const double kstep_us[4] = {0.559, 0.311, 0.310, 0.304}, wave_us[4] = {8.05, 5.32, 4.02, 4.14};
            auto model = [&](uint32_t ti, uint32_t c, uint32_t* eff_out) {
                const uint32_t tt = 512u >> ti;
                const uint32_t mt = (m + tt - 1u) / tt;
                const uint32_t rbs = (raw_blocks + c - 1u) / c, eff = (raw_blocks + rbs - 1u) / rbs;
                const double waves = static_cast<double>((mt * n_pairs * eff + sm_pairs - 1u) / sm_pairs);
                double us = 4.51 + waves * (rbs * 4.0 * kstep_us[ti] + wave_us[ti]);
                if (eff > 1u) us += -1.12 + static_cast<double>(eff) * m * n * 4.0 / 3.33e6;
                *eff_out = eff;
                return us;
            };
            double best = 1e30;
            uint32_t best_tt = p->tm, best_c = splits;
            for (uint32_t ti = 0; ti < 4u; ti++) {
                const uint32_t tt = 512u >> ti;
                if (s.tm ? tt != s.tm : (tt != 64u && tt / 2u >= m)) continue;      // the caller's tile; or no tile more than half empty
                for (uint32_t c = 1; c <= 8u && (c == 1u || raw_blocks / c >= 4u); c++) {
                    if (s.k_splits && c != s.k_splits) continue;                    // the caller fixed the splits
                    uint32_t eff = 0;
                    const double us = model(ti, c, &eff);
                    if (eff != c && !s.k_splits) continue;                          // the same plan as a smaller c
                    if (us < best * 0.98) {
                        best = us;
                        best_tt = tt;
                        best_c = c;
                    }
                }
            }
            splits = best_c;
            p->tm = best_tt;
            p->tok_blocks = best_tt == 512u ? 2u : 1u;
            p->m_tiles = (m + p->tm - 1u) / p->tm;
        }
        p->x_rows = p->tm == 512u ? lexb::PAIR_XBLK_ROWS : p->tm / 2u;
        // packed-weight blocks in flight: 2; 3 with tiles of 128 tokens or fewer, whose K step is short enough for the
        // third block's trip to HBM to show (2-3 % per launch)
        const uint32_t raw_stages = env_u32("LEXB_RAWSTAGES", p->tm <= 128u ? 3u : lexb::PAIR_RAW_STAGES);
        p->raw_stages = raw_stages;
        if (splits < 1u || splits > raw_blocks) return bail(fail(LEXB_ERR_ARG, "k_splits = %u outside [1, %u]", splits, raw_blocks));
        // Ring depths.  Tiles of 512 tokens: x ring of 4 stages of 32 KiB, W ring of 3 of 16 KiB, two packed-weight
        // blocks: 212 KiB; their K step is bound by the MMAs.  Smaller tiles: a K step's MMAs take half as long or
        // less and the shared-memory pipe would set the pace, so the decoded W tiles go to tensor memory (the columns
        // behind the accumulator: 256 with tiles of 256 tokens, 384 below; 32 columns per K step) and the MMAs read
        // them from there.  A ring stage then holds two K steps (x 2 x 16 KiB with 256 tokens, W 64 columns; x ring of
        // 4, W ring of 4 or 6) or, with tiles of 128 tokens or fewer, a whole block of four (x ring of 3, W ring of 3),
        // and the MMA warp waits and commits once per stage.  Depths the caller gives that do not fit that way are
        // taken as stages of one K step (at most 8 W stages in tensor memory); more than 8 W stages, or
        // LEXB_WTMEM=0, put the W ring in shared memory (x 6, W 5 by default).
        const bool w_tmem = p->tok_blocks == 1u && s.w_stages <= 8u && env_u32("LEXB_WTMEM", 1u) != 0u;
        uint32_t k_sub = w_tmem ? env_u32("LEXB_KSUB", p->x_rows <= 64u ? 4u : 2u) : 1u;
        if (k_sub != 1u && k_sub != 2u && k_sub != 4u) k_sub = 1u;
        const uint32_t w_cols = p->x_rows <= 64u ? 384u : 256u;             // TMEM columns behind the accumulator
        const uint32_t w_max = k_sub ? w_cols / (32u * k_sub) : 0u;
        if (k_sub > 1u && (s.w_stages > w_max ||
                            lexb::pair_smem_bytes(1u, s.stages ? s.stages : (k_sub == 4u ? 2u : 4u), 2u, raw_stages, true, k_sub, p->x_rows) > g->smem_optin))
            k_sub = 1u;
        const uint32_t stages = s.stages ? s.stages : (p->tok_blocks == 2u ? 4u : k_sub == 4u ? (p->x_rows == 128u ? 2u : 3u) : k_sub == 2u ? 4u : w_tmem ? 8u : 6u);
        const uint32_t w_stages = s.w_stages ? s.w_stages : (p->tok_blocks == 2u ? 3u : k_sub >= 2u ? w_cols / (32u * k_sub) : w_tmem ? 8u : 5u);
        const uint32_t need = lexb::pair_smem_bytes(p->tok_blocks, stages, w_stages, raw_stages, w_tmem, k_sub, p->x_rows);
        if (stages < 2 || w_stages < 2 || raw_stages < 2 || need > g->smem_optin)
            return bail(fail(LEXB_ERR_ARG, "stages = %u with w_stages = %u and %u packed-weight blocks need %u bytes of shared memory (limit %zu)",
                             stages, w_stages, raw_stages, need, g->smem_optin));
        p->k_sub = k_sub;
        p->stages = stages; p->w_stages = w_stages;
        if (w_tmem) p->flags |= 4u;
        const uint32_t tiles_final = p->m_tiles * n_pairs;
        const uint32_t rb_per_split = (raw_blocks + splits - 1u) / splits;
        splits = (raw_blocks + rb_per_split - 1u) / rb_per_split;          // no empty split
        p->k_splits = splits;
        p->kb_per_split = rb_per_split * (lexb::PAIR_RAW_K / lexb::GEMM_BK);
        if (splits > 1u) {
            cudaError_t e = x_malloc(&p->partial, sizeof(float) * splits * static_cast<size_t>(m) * n);
            if (e != cudaSuccess) return bail(fail(LEXB_ERR_CUDA, "allocating the split-K workspace: %s", cudaGetErrorString(e)));
        }
        p->grid = 2u * tiles_final * splits;
        p->threads = lexb::PAIR_THREADS;
        p->smem = need;
        snprintf(p->entry, sizeof p->entry, "%s_%u_%u_%u_%u_%u_%u", stem, m, n, k, p->tm, 2u * lexb::GEMM_TN, lexb::GEMM_BK);
    } else {
        if (n % lexb::MV_ROWS) return bail(fail(LEXB_ERR_SHAPE, "gemm_fp4 (matvec): %u rows per block do not divide n = %u", lexb::MV_ROWS, n));
        if (k % 32u) return bail(fail(LEXB_ERR_SHAPE, "gemm_fp4 (matvec): 32 does not divide k = %u", k));
        uint32_t kc = s.kc;
        if (!kc) {
            // the whole of K if x fits in 96 KiB of shared memory (blocks are then persistent and
            // stage x once), else the largest multiple of one block round (1024 columns) that does
            const uint32_t budget = 98304u;
            kc = round_up(k, lexb::MV_ROUND);
            while (kc > lexb::MV_ROUND && m * lexb::matvec_x_pitch(kc) > budget) kc -= lexb::MV_ROUND;
        }
        if (kc % lexb::MV_ROUND || kc == 0) return bail(fail(LEXB_ERR_ARG, "kc = %u is not a multiple of %u", kc, lexb::MV_ROUND));
        p->kc = kc;
        p->threads = lexb::MV_THREADS;
        p->smem = lexb::matvec_smem_bytes(m, kc, lexb::matvec_uses_ring(m));
        if (p->smem > g->smem_optin) return bail(fail(LEXB_ERR_UNSUPPORTED, "kc = %u needs %u bytes of shared memory", kc, p->smem));
        const uint32_t row_blocks = n / lexb::MV_ROWS;
        if (kc >= k) {
            // persistent: as many blocks as stay resident (4 per SM by registers), each with the same
            // number of row blocks
            uint32_t per_sm = static_cast<uint32_t>(g->smem_optin / (p->smem + 1024u));
            if (per_sm > 4u) per_sm = 4u;
            if (per_sm < 1u) per_sm = 1u;
            const uint32_t max_blocks = per_sm * static_cast<uint32_t>(g->prop.multiProcessorCount);
            const uint32_t per_block = (row_blocks + max_blocks - 1u) / max_blocks;
            p->grid = (row_blocks + per_block - 1u) / per_block;
        } else {
            p->grid = row_blocks;
        }
        snprintf(p->entry, sizeof p->entry, "%s_%u_%u_%u_%u_%u_%u", stem, m, n, k, m, lexb::MV_ROWS, lexb::MV_SLICE);
    }
    *out = p;
    return LEXB_OK;
}

int lexb_matmul_fp4_plan(lexb_gpu* g, uint32_t t, uint32_t n_out, uint32_t n_in, int residual, int x_half,
                         const lexb_sched* sched, lexb_pipeline** out) {
    if (!out) return fail(LEXB_ERR_ARG, "lexb_matmul_fp4_plan: null out");
    *out = nullptr;
    lexb_sched s{};
    if (sched) s = *sched;
    s.kernel = KERNEL_MATMUL_Q;
    int rc = lexb_gemm_fp4_plan(g, t, n_out, n_in, residual, &s, out);
    if (rc) return rc;
    // the reference's name for the program: matvec / matmul{t}, layout tag, rows x columns, _res, _xh
    // (crates/lex-front/src/llama.rs:416-422, :459-465)
    char tag[16];
    if (t == 1) snprintf(tag, sizeof tag, "matvec");
    else snprintf(tag, sizeof tag, "matmul%u", t);
    (*out)->x_f32 = !x_half;
    snprintf((*out)->entry, sizeof (*out)->entry, "%s_nvfp4_%ux%u%s%s", tag, n_out, n_in, residual ? "_res" : "", x_half ? "_xh" : "");
    return LEXB_OK;
}

int lexb_matmul_int8_plan(lexb_gpu* g, uint32_t t, uint32_t n_out, uint32_t n_in, int residual, const lexb_sched* sched,
                          lexb_pipeline** out) {
    if (!out) return fail(LEXB_ERR_ARG, "lexb_matmul_int8_plan: null out");
    *out = nullptr;
    lexb_sched s{};
    if (sched) s = *sched;
    s.kernel = KERNEL_MATMUL_Q;
    t_plan_q16 = true;
    int rc = lexb_gemm_fp4_plan(g, t, n_out, n_in, residual, &s, out);
    t_plan_q16 = false;
    if (rc) return rc;
    // the reference's name for the kernel (crates/lex-msl/src/int8.rs:129-132)
    snprintf((*out)->entry, sizeof (*out)->entry, "matmul_int8_%ux%ux%u%s", t, n_out, n_in, residual ? "_res" : "");
    return LEXB_OK;
}

int lexb_quant16(lexb_gpu* g, uint32_t m, uint32_t k, int x_half, const lexb_buffer* x, lexb_buffer* xq, lexb_buffer* xs) {
    int rc = use(g);
    if (rc) return rc;
    if (m == 0 || k == 0 || k % 32u) return fail(LEXB_ERR_SHAPE, "quant16: %u inputs are not whole groups of 32", k);
    const size_t mm = m, kk = k;
    if ((rc = check_buf(x, g, mm * kk * (x_half ? 2 : 4), "x"))) return rc;
    if ((rc = check_buf(xq, g, mm * kk * 2, "xq"))) return rc;
    if ((rc = check_buf(xs, g, mm * (kk / 16) * 4, "xs"))) return rc;
    const size_t groups = mm * kk / 16;
    const uint32_t blocks = static_cast<uint32_t>((groups + 255) / 256);
    INJECT_LAUNCH();
    if (x_half) quant16_kernel<true><<<blocks, 256, 0, g->stream>>>(x->ptr, static_cast<short*>(xq->ptr), static_cast<float*>(xs->ptr), groups);
    else quant16_kernel<false><<<blocks, 256, 0, g->stream>>>(x->ptr, static_cast<short*>(xq->ptr), static_cast<float*>(xs->ptr), groups);
    CUDA_TRY(cudaGetLastError());
    return LEXB_OK;
}

void lexb_pipeline_free(lexb_pipeline* p) {
    if (!p) return;
    if (p->partial || p->pre_buf) {
        cudaSetDevice(p->gpu->device);
        cudaFree(p->partial);
        cudaFree(p->pre_buf);
    }
    delete p;
}

int lexb_pipeline_describe(const lexb_pipeline* p, lexb_lowered* out) {
    if (!p || !out) return fail(LEXB_ERR_ARG, "lexb_pipeline_describe: null argument");
    memset(out, 0, sizeof *out);
    snprintf(out->entry, sizeof out->entry, "%s", p->entry);
    out->grid = p->grid;
    out->grid2 = 1;
    out->threads = p->threads;
    out->threadgroup_bytes = p->smem;
    out->nbind = (p->residual ? 6 : 5) + (p->x_q16 ? 1 : 0);
    out->writes[out->nbind - 1] = 1;
    out->kernel = p->kernel;
    out->m = p->m; out->n = p->n; out->k = p->k; out->residual = p->residual;
    if (p->kernel == KERNEL_MATMUL_Q) {
        out->bm = p->m; out->bn = lexb::MQ_ROWS; out->bk = lexb::MQ_STAGE_K; out->stages = p->stages;
        out->k_splits = p->k_splits;
        out->scratch_bytes = p->partial ? sizeof(float) * p->k_splits * static_cast<uint64_t>(p->m) * p->n : 0;
    } else if (p->kernel == KERNEL_TCGEN05 || p->kernel == KERNEL_TCGEN05_PAIR) {
        out->bm = p->tm; out->bn = p->kernel == KERNEL_TCGEN05_PAIR ? 2u * lexb::GEMM_TN : lexb::GEMM_TN;
        out->bk = lexb::GEMM_BK; out->stages = p->stages;
        out->k_splits = p->k_splits;
        out->scratch_bytes = p->partial ? sizeof(float) * p->k_splits * static_cast<uint64_t>(p->m) * p->n : 0;
    } else {
        out->bm = p->m; out->bn = lexb::MV_ROWS; out->bk = lexb::MV_SLICE; out->stages = 1;
    }
    return LEXB_OK;
}

int lexb_gemm_fp4_launch(lexb_gpu* g, const lexb_pipeline* p, const lexb_buffer* x, const lexb_buffer* wq,
                         const lexb_buffer* ws, const lexb_buffer* wg, const lexb_buffer* r, lexb_buffer* y) {
    int rc = use(g);
    if (rc) return rc;
    return launch_one(g, p, x, wq, ws, wg, r, y);
}

int lexb_gemm_fp4_launch_gather(lexb_gpu* g, const lexb_pipeline* p, const lexb_buffer* x, const lexb_buffer* wq,
                                const lexb_buffer* ws, const lexb_buffer* wg, const lexb_buffer* r, void* const* y_of_rank,
                                uint32_t world, uint32_t n_total, uint32_t n0) {
    int rc = use(g);
    if (rc) return rc;
    if (!p || !y_of_rank) return fail(LEXB_ERR_ARG, "lexb_gemm_fp4_launch_gather: null argument");
    if (world == 0 || world > lexb::GATHER_MAX) return fail(LEXB_ERR_ARG, "world = %u outside [1, %u]", world, lexb::GATHER_MAX);
    if (n_total % 4u || n0 % 4u || static_cast<uint64_t>(n0) + p->n > n_total)
        return fail(LEXB_ERR_ARG, "columns [%u, %u) do not fit a gathered row of %u", n0, n0 + p->n, n_total);
    lexb::GatherDst gd{};
    gd.world = world; gd.n_total = n_total; gd.n0 = n0; gd.n_local = p->n;
    for (uint32_t d = 0; d < world; d++) {
        if (!y_of_rank[d] || (reinterpret_cast<uintptr_t>(y_of_rank[d]) & 15u))
            return fail(LEXB_ERR_ARG, "y of rank %u is null or not 16-byte aligned", d);
        gd.y[d] = static_cast<float*>(y_of_rank[d]);
    }
    return launch_one(g, p, x, wq, ws, wg, r, nullptr, &gd);
}

int lexb_gemm_fp4_silu_launch(lexb_gpu* g, const lexb_pipeline* p, const lexb_buffer* x, const lexb_buffer* wq,
                              const lexb_buffer* ws, const lexb_buffer* wg, lexb_buffer* act) {
    int rc = use(g);
    if (rc) return rc;
    if (!act) return fail(LEXB_ERR_ARG, "lexb_gemm_fp4_silu_launch: null act");
    return launch_one(g, p, x, wq, ws, wg, nullptr, nullptr, nullptr, nullptr, Order{}, act);
}

int lexb_gemm_fp4_silu_launch_gather(lexb_gpu* g, const lexb_pipeline* p, const lexb_buffer* x, const lexb_buffer* wq,
                                     const lexb_buffer* ws, const lexb_buffer* wg, void* const* act_of_rank, uint32_t world,
                                     uint32_t n_total, uint32_t n0) {
    int rc = use(g);
    if (rc) return rc;
    if (!p || !act_of_rank) return fail(LEXB_ERR_ARG, "lexb_gemm_fp4_silu_launch_gather: null argument");
    if (world == 0 || world > lexb::GATHER_MAX) return fail(LEXB_ERR_ARG, "world = %u outside [1, %u]", world, lexb::GATHER_MAX);
    if (n_total % 8u || n0 % 8u || static_cast<uint64_t>(n0) + p->n > n_total)
        return fail(LEXB_ERR_ARG, "interleaved rows [%u, %u) do not fit %u rows in all", n0, n0 + p->n, n_total);
    lexb::GatherDst gd{};
    gd.world = world; gd.n_total = n_total; gd.n0 = n0; gd.n_local = p->n; gd.silu = 1u;
    for (uint32_t d = 0; d < world; d++) {
        if (!act_of_rank[d] || (reinterpret_cast<uintptr_t>(act_of_rank[d]) & 15u))
            return fail(LEXB_ERR_ARG, "act of rank %u is null or not 16-byte aligned", d);
        gd.y[d] = static_cast<float*>(act_of_rank[d]);
    }
    return launch_one(g, p, x, wq, ws, wg, nullptr, nullptr, &gd);
}

int lexb_interleave_rows(lexb_gpu* g, const lexb_buffer* a, const lexb_buffer* b, size_t rows, size_t row_bytes, lexb_buffer* out) {
    int rc = use(g);
    if (rc) return rc;
    if (!a || !b || !out) return fail(LEXB_ERR_ARG, "lexb_interleave_rows: null buffer");
    if (rows == 0 || row_bytes == 0) return fail(LEXB_ERR_SHAPE, "lexb_interleave_rows: empty extent");
    if (a->bytes < rows * row_bytes || b->bytes < rows * row_bytes || out->bytes < 2 * rows * row_bytes)
        return fail(LEXB_ERR_ARG, "lexb_interleave_rows: %zu rows of %zu bytes do not fit the buffers", rows, row_bytes);
    char* o = static_cast<char*>(out->ptr);
    CUDA_TRY_AT(SITE_COPY, cudaMemcpy2DAsync(o, 2 * row_bytes, a->ptr, row_bytes, row_bytes, rows, cudaMemcpyDeviceToDevice, g->stream));
    CUDA_TRY_AT(SITE_COPY, cudaMemcpy2DAsync(o + row_bytes, 2 * row_bytes, b->ptr, row_bytes, row_bytes, rows, cudaMemcpyDeviceToDevice, g->stream));
    return LEXB_OK;
}

int lexb_gemm_fp4_enqueue_host(lexb_gpu* g, const lexb_pipeline* p, const void* x_host, lexb_buffer* x_dev,
                               const lexb_buffer* wq, const lexb_buffer* ws, const lexb_buffer* wg, const lexb_buffer* r,
                               lexb_buffer* y_dev, void* y_host) {
    int rc = use(g);
    if (rc) return rc;
    if (!p || !x_host || !y_host || !x_dev || !y_dev) return fail(LEXB_ERR_ARG, "lexb_gemm_fp4_enqueue_host: null argument");
    if (p->x_q16) return fail(LEXB_ERR_UNSUPPORTED, "lexb_gemm_fp4_enqueue_host takes f16 or f32 activations; quantise on the device (lexb_quant16) and launch a step");
    const size_t xb = static_cast<size_t>(p->m) * p->k * (p->x_f32 ? 4 : 2), yb = static_cast<size_t>(p->m) * p->n * 4;
    if (x_dev->bytes < xb || y_dev->bytes < yb) return fail(LEXB_ERR_ARG, "lexb_gemm_fp4_enqueue_host: staging buffers too small");
    CUDA_TRY_AT(SITE_COPY, cudaMemcpyAsync(x_dev->ptr, x_host, xb, cudaMemcpyHostToDevice, g->stream));
    if ((rc = launch_one(g, p, x_dev, wq, ws, wg, r, y_dev))) return rc;
    CUDA_TRY_AT(SITE_COPY, cudaMemcpyAsync(y_host, y_dev->ptr, yb, cudaMemcpyDeviceToHost, g->stream));
    return LEXB_OK;
}

int lexb_gemm_fp4_run_host(lexb_gpu* g, const lexb_pipeline* p, const void* x_host, lexb_buffer* x_dev,
                           const lexb_buffer* wq, const lexb_buffer* ws, const lexb_buffer* wg, const lexb_buffer* r,
                           lexb_buffer* y_dev, void* y_host) {
    int rc = use(g);
    if (rc) return rc;
    if (!p || !x_host || !y_host || !x_dev || !y_dev) return fail(LEXB_ERR_ARG, "lexb_gemm_fp4_run_host: null argument");
    if (p->x_q16) return fail(LEXB_ERR_UNSUPPORTED, "lexb_gemm_fp4_run_host takes f16 or f32 activations; quantise on the device (lexb_quant16) and launch a step");
    const size_t xb = static_cast<size_t>(p->m) * p->k * (p->x_f32 ? 4 : 2), yb = static_cast<size_t>(p->m) * p->n * 4;
    if (x_dev->bytes < xb || y_dev->bytes < yb) return fail(LEXB_ERR_ARG, "lexb_gemm_fp4_run_host: staging buffers too small");
    CUDA_TRY_AT(SITE_COPY, cudaMemcpyAsync(x_dev->ptr, x_host, xb, cudaMemcpyHostToDevice, g->stream));
    if ((rc = launch_one(g, p, x_dev, wq, ws, wg, r, y_dev))) return rc;
    CUDA_TRY_AT(SITE_COPY, cudaMemcpyAsync(y_host, y_dev->ptr, yb, cudaMemcpyDeviceToHost, g->stream));
    CUDA_TRY(cudaStreamSynchronize(g->stream));
    return LEXB_OK;
}

int lexb_run_launches(lexb_gpu* g, const lexb_step* steps, size_t nsteps, double* cpu_s, double* wall_s) {
    int rc = use(g);
    if (rc) return rc;
    if (!steps && nsteps) return fail(LEXB_ERR_ARG, "lexb_run_launches: null steps");
    const auto t0 = std::chrono::steady_clock::now();
    ListProof proof;
    bool first = true;
    if ((rc = issue_list(g, steps, nsteps, proof, first, nullptr))) return rc;
    const auto t1 = std::chrono::steady_clock::now();
    CUDA_TRY(cudaStreamSynchronize(g->stream));
    const auto t2 = std::chrono::steady_clock::now();
    if (cpu_s) *cpu_s = std::chrono::duration<double>(t1 - t0).count();
    if (wall_s) *wall_s = std::chrono::duration<double>(t2 - t0).count();
    return LEXB_OK;
}

int lexb_run_each_timed(lexb_gpu* g, const lexb_step* steps, size_t nsteps, double* seconds_out) {
    int rc = use(g);
    if (rc) return rc;
    if ((!steps || !seconds_out) && nsteps) return fail(LEXB_ERR_ARG, "lexb_run_each_timed: null argument");
    std::vector<cudaEvent_t> ev(nsteps + 1, nullptr);
    auto cleanup = [&]() { for (auto e : ev) if (e) cudaEventDestroy(e); };
    for (auto& e : ev)
        if (cudaEventCreate(&e) != cudaSuccess) { cleanup(); return fail(LEXB_ERR_CUDA, "cudaEventCreate failed"); }
    cudaEventRecord(ev[0], g->stream);
    ListProof proof;
    for (size_t i = 0; i < nsteps; i++) {
        const StepRanges sr = step_ranges(steps[i]);
        Order order;
        order.fence = i == 0;
        order.early_weights = sr.valid && proof.weights_untouched(sr);
        if ((rc = launch_step(g, steps[i], i + 1 < nsteps ? &steps[i + 1] : nullptr, order))) { cleanup(); return rc; }
        if (sr.valid) proof.add(sr);
        cudaEventRecord(ev[i + 1], g->stream);
    }
    cudaError_t e = cudaStreamSynchronize(g->stream);
    if (e != cudaSuccess) { cleanup(); return fail(LEXB_ERR_CUDA, "synchronise: %s", cudaGetErrorString(e)); }
    for (size_t i = 0; i < nsteps; i++) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, ev[i], ev[i + 1]);
        seconds_out[i] = ms * 1e-3;
    }
    cleanup();
    return LEXB_OK;
}

int lexb_list_runs(lexb_gpu* g, const lexb_step* steps, size_t nsteps, uint32_t* run_len_out) {
    int rc = use(g);
    if (rc) return rc;
    if ((!steps || !run_len_out) && nsteps) return fail(LEXB_ERR_ARG, "lexb_list_runs: null argument");
    ListProof proof;
    for (size_t i = 0; i < nsteps;) {
        const size_t len = chain_run(g, steps, nsteps, i, proof);
        const size_t take = len ? len : 1;
        for (size_t e = i; e < i + take; e++) {
            run_len_out[e] = static_cast<uint32_t>(take);
            const StepRanges sr = step_ranges(steps[e]);
            if (sr.valid) proof.add(sr);
        }
        i += take;
    }
    return LEXB_OK;
}

int lexb_time_launches(lexb_gpu* g, const lexb_step* steps, size_t nsteps, uint32_t reps, double* seconds_out) {
    int rc = use(g);
    if (rc) return rc;
    if ((!steps && nsteps) || !seconds_out) return fail(LEXB_ERR_ARG, "lexb_time_launches: null argument");
    cudaEvent_t a, b;
    CUDA_TRY(cudaEventCreate(&a));
    CUDA_TRY(cudaEventCreate(&b));
    CUDA_TRY(cudaStreamSynchronize(g->stream));
    cudaEventRecord(a, g->stream);
    ListProof proof;
    bool first = true;
    for (uint32_t r = 0; r < reps; r++) {
        // the list repeats: the step after the last one is the first one again
        const lexb_step* after_last = (r + 1 < reps && nsteps) ? &steps[0] : nullptr;
        if ((rc = issue_list(g, steps, nsteps, proof, first, after_last))) { cudaEventDestroy(a); cudaEventDestroy(b); return rc; }
    }
    cudaEventRecord(b, g->stream);
    cudaError_t e = cudaStreamSynchronize(g->stream);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, a, b);
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    if (e != cudaSuccess) return fail(LEXB_ERR_CUDA, "timing: %s", cudaGetErrorString(e));
    *seconds_out = ms * 1e-3;
    return LEXB_OK;
}

int lexb_status_word(lexb_gpu* g, uint32_t* out) {
    int rc = use(g);
    if (rc) return rc;
    if (!out) return fail(LEXB_ERR_ARG, "lexb_status_word: null out");
    // read and cleared in the launch stream's order, then waited for: the legacy default stream would not be
    // ordered with the library's non-blocking stream
    CUDA_TRY(cudaMemcpyAsync(out, g->d_status, sizeof(uint32_t), cudaMemcpyDeviceToHost, g->stream));
    CUDA_TRY(cudaMemsetAsync(g->d_status, 0, sizeof(uint32_t), g->stream));
    CUDA_TRY(cudaStreamSynchronize(g->stream));
    return LEXB_OK;
}

int lexb_trace_enable(lexb_gpu* g, uint32_t max_ctas) {
    int rc = use(g);
    if (rc) return rc;
    if (g->d_trace) {
        CUDA_TRY(cudaFree(g->d_trace));
        g->d_trace = nullptr;
        g->trace_ctas = 0;
    }
    if (max_ctas) {
        CUDA_TRY(x_malloc(&g->d_trace, sizeof(unsigned long long) * 16u * max_ctas));
        CUDA_TRY(cudaMemsetAsync(g->d_trace, 0, sizeof(unsigned long long) * 16u * max_ctas, g->stream));
        CUDA_TRY(cudaStreamSynchronize(g->stream));
        g->trace_ctas = max_ctas;
    }
    return LEXB_OK;
}

int lexb_trace_read(lexb_gpu* g, uint64_t* out, uint32_t ctas) {
    int rc = use(g);
    if (rc) return rc;
    if (!out || !g->d_trace || ctas > g->trace_ctas) return fail(LEXB_ERR_ARG, "lexb_trace_read: tracing is off or the request is too large");
    CUDA_TRY(cudaMemcpyAsync(out, g->d_trace, sizeof(uint64_t) * 16u * ctas, cudaMemcpyDeviceToHost, g->stream));
    CUDA_TRY(cudaStreamSynchronize(g->stream));
    return LEXB_OK;
}

int lexb_selftest_bounded_wait(lexb_gpu* g, uint32_t limit_us) {
    int rc = use(g);
    if (rc) return rc;
    if (limit_us == 0 || limit_us > 1000000u) return fail(LEXB_ERR_ARG, "limit_us must be in [1, 1000000]");
    const long long cycles = static_cast<long long>(limit_us) * (g->prop.clockRate / 1000);   // clockRate is kHz
    INJECT_LAUNCH();
    bounded_wait_selftest_kernel<<<1, 32, 0, g->stream>>>(g->d_status, cycles);
    CUDA_TRY(cudaGetLastError());
    CUDA_TRY(cudaStreamSynchronize(g->stream));
    return LEXB_OK;
}

int lexb_dequant_fp4_f16(lexb_gpu* g, uint32_t n, uint32_t k, const lexb_buffer* wq, const lexb_buffer* ws,
                         const lexb_buffer* wg, lexb_buffer* w_f16) {
    int rc = use(g);
    if (rc) return rc;
    if (n == 0 || k == 0 || k % 16u) return fail(LEXB_ERR_SHAPE, "dequant_fp4: group 16 does not divide k = %u", k);
    const size_t nn = n, kk = k;
    if ((rc = check_buf(wq, g, nn * kk / 2, "wq"))) return rc;
    if ((rc = check_buf(ws, g, nn * kk / 16, "ws"))) return rc;
    if ((rc = check_buf(wg, g, nn * 4, "wg"))) return rc;
    if ((rc = check_buf(w_f16, g, nn * kk * 2, "w_f16"))) return rc;
    const size_t groups = nn * kk / 16;
    const uint32_t threads = 256;
    const uint32_t blocks = static_cast<uint32_t>(std::min<size_t>((groups + threads - 1) / threads, static_cast<size_t>(g->prop.multiProcessorCount) * 32u));
    INJECT_LAUNCH();
    dequant_fp4_f16_kernel<<<blocks, threads, 0, g->stream>>>(n, k, static_cast<const uint8_t*>(wq->ptr),
                                                              static_cast<const uint8_t*>(ws->ptr),
                                                              static_cast<const float*>(wg->ptr),
                                                              static_cast<uint16_t*>(w_f16->ptr));
    CUDA_TRY(cudaGetLastError());
    return LEXB_OK;
}

int lexb_gemm_fp4_splitk_static(lexb_gpu* g, uint32_t m, uint32_t n, uint32_t k, uint32_t k_splits, const lexb_buffer* x,
                                const lexb_buffer* wq, const lexb_buffer* ws, const lexb_buffer* wg, const lexb_buffer* r,
                                lexb_buffer* y) {
    int rc = use(g);
    if (rc) return rc;
    if (m < lexb::PAIR_XBLK_ROWS || n == 0 || n % lexb::GEMM_TN || k == 0 || k % lexb::PAIR_RAW_K)
        return fail(LEXB_ERR_SHAPE, "gemm_fp4 (static scratch): needs m >= %u, n %% %u == 0, k %% %u == 0; got m=%u n=%u k=%u",
                    lexb::PAIR_XBLK_ROWS, lexb::GEMM_TN, lexb::PAIR_RAW_K, m, n, k);
    const uint32_t raw_blocks = k / lexb::PAIR_RAW_K;
    if (k_splits < 2u || k_splits > 8u || k_splits > raw_blocks)
        return fail(LEXB_ERR_ARG, "k_splits = %u outside [2, %u]", k_splits, raw_blocks < 8u ? raw_blocks : 8u);
    const uint32_t rb_per_split = (raw_blocks + k_splits - 1u) / k_splits;
    const uint32_t splits = (raw_blocks + rb_per_split - 1u) / rb_per_split;
    const uint64_t need = sizeof(float) * static_cast<uint64_t>(splits) * m * n;
    if (need > LEXB_STATIC_SCRATCH_BYTES)
        return fail(LEXB_ERR_UNSUPPORTED,
                    "gemm_fp4 (static scratch): %u splits of m=%u n=%u need %llu bytes of scratch, the built-in array holds %llu; "
                    "use fewer splits or a planned pipeline",
                    splits, m, n, (unsigned long long)need, (unsigned long long)LEXB_STATIC_SCRATCH_BYTES);
    if (!g->static_scratch) {
        // Once per device, with that device current (use() above): the symbol's name is a host-side
        // stand-in, the kernels need its device address.
        void* p = nullptr;
        CUDA_TRY(cudaGetSymbolAddress(&p, g_splitk_static_scratch));
        g->static_scratch = static_cast<float*>(p);
    }
    // The same launch shape lexb_gemm_fp4_plan builds for the two-CTA kernel, held on the stack.
    lexb_pipeline p;
    p.gpu = g;
    p.kernel = KERNEL_TCGEN05_PAIR;
    p.m = m; p.n = n; p.k = k;
    p.residual = r != nullptr;
    // one block of 256 tokens per tile up to m = 256, two beyond: the shape lexb_gemm_fp4_plan gives the same m
    p.tok_blocks = m > 256u ? 2u : 1u;
    p.tm = p.tok_blocks * 256u; p.stages = 4; p.w_stages = 3; p.tmem_cols = lexb::PAIR_TMEM_COLS; p.n_acc = 1; p.flags = 0;
    p.kc = 0;
    p.m_tiles = (m + p.tm - 1) / p.tm;
    p.k_splits = splits;
    p.kb_per_split = rb_per_split * (lexb::PAIR_RAW_K / lexb::GEMM_BK);
    p.grid = 2u * p.m_tiles * ((n + 2u * lexb::GEMM_TN - 1) / (2u * lexb::GEMM_TN)) * splits;
    p.threads = lexb::PAIR_THREADS;
    p.smem = lexb::pair_smem_bytes(2u, p.stages, p.w_stages);
    if (p.smem > g->smem_optin) return fail(LEXB_ERR_UNSUPPORTED, "the device offers %zu bytes of shared memory, the kernel needs %u", g->smem_optin, p.smem);
    const size_t mm = m, nn = n, kk = k;
    if ((rc = check_buf(x, g, mm * kk * 2, "x"))) return rc;
    if ((rc = check_buf(wq, g, nn * kk / 2, "wq"))) return rc;
    if ((rc = check_buf(ws, g, nn * kk / 16, "ws"))) return rc;
    if ((rc = check_buf(wg, g, nn * 4, "wg"))) return rc;
    if ((rc = check_buf(y, g, mm * nn * 4, "y"))) return rc;
    if (r && (rc = check_buf(r, g, mm * nn * 4, "r"))) return rc;
    CUtensorMap map_x, map_wq, map_ws;      // encoded on the host for this call, not cached
    if ((rc = encode_2d(&p, &map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x->ptr, k, m, lexb::GEMM_BK, lexb::PAIR_XBLK_ROWS,
                        CU_TENSOR_MAP_SWIZZLE_128B, "x")))
        return rc;
    if ((rc = encode_2d(&p, &map_wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq->ptr, k / 2, n, lexb::PAIR_RAW_K / 2, lexb::GEMM_TN,
                        CU_TENSOR_MAP_SWIZZLE_128B, "wq")))
        return rc;
    if ((rc = encode_2d(&p, &map_ws, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, ws->ptr, k / 16, n, lexb::PAIR_RAW_K / 16, lexb::GEMM_TN,
                        CU_TENSOR_MAP_SWIZZLE_NONE, "ws")))
        return rc;
    lexb::GemmArgs a{};
    a.wq = static_cast<const uint8_t*>(wq->ptr);
    a.ws = static_cast<const uint8_t*>(ws->ptr);
    a.wg = static_cast<const float*>(wg->ptr);
    a.r = r ? static_cast<const float*>(r->ptr) : nullptr;
    a.y = static_cast<float*>(y->ptr);
    a.status = g->d_status;
    a.trace = nullptr;
    a.m = m; a.n = n; a.k = k;
    a.tm = p.tm; a.stages = p.stages; a.w_stages = p.w_stages; a.raw_stages = p.raw_stages; a.k_sub = 1; a.x_rows = lexb::PAIR_XBLK_ROWS;
    a.flags = p.tok_blocks == 1u ? 4u : 0u;      // tiles of 256 tokens: W tiles in tensor memory, as the planned pipeline has them
    a.k_splits = splits; a.kb_per_split = p.kb_per_split; a.tok_blocks = p.tok_blocks;
    a.partial = g->static_scratch;          // every element of the partials is written before it is read: nothing to clear
    a.tmem_cols = p.tmem_cols; a.m_tiles = p.m_tiles; a.n_acc = 1;
    a.x_tx_bytes = lexb::PAIR_XBLK_BYTES;
    INJECT_LAUNCH();
    lexb::gemm_fp4_tcgen05_pair_kernel<false><<<p.grid, p.threads, p.smem, g->stream>>>(map_x, map_wq, map_ws, a);
    CUDA_TRY(cudaGetLastError());
    const size_t elems = mm * nn;
    const uint32_t blocks = static_cast<uint32_t>(std::min<size_t>((elems / 4 + 255) / 256, static_cast<size_t>(g->prop.multiProcessorCount) * 8u));
    INJECT_LAUNCH();
    lexb::splitk_reduce_kernel<<<blocks, 256, 0, g->stream>>>(g->static_scratch, splits, elems, a.r, a.y, lexb::GatherDst{},
                                                              static_cast<uint16_t*>(nullptr), n);
    CUDA_TRY(cudaGetLastError());
    return LEXB_OK;
}

int lexb_silu_mul(lexb_gpu* g, uint32_t rows, uint32_t cols, const lexb_buffer* gate, size_t gate_offset, size_t gate_pitch,
                  const lexb_buffer* up, size_t up_offset, size_t up_pitch, lexb_buffer* out, int out_f16) {
    int rc = use(g);
    if (rc) return rc;
    if (!gate || !up || !out) return fail(LEXB_ERR_ARG, "lexb_silu_mul: null buffer");
    if (rows == 0 || cols == 0 || cols % 4u) return fail(LEXB_ERR_SHAPE, "silu_mul: 4 must divide cols = %u", cols);
    if (gate_pitch < cols || up_pitch < cols || (gate_pitch | up_pitch | gate_offset | up_offset) % 4u)
        return fail(LEXB_ERR_ARG, "silu_mul: pitches and offsets are in f32 elements, multiples of 4, pitch >= cols");
    const size_t need_g = (gate_offset + static_cast<size_t>(rows - 1) * gate_pitch + cols) * 4;
    const size_t need_u = (up_offset + static_cast<size_t>(rows - 1) * up_pitch + cols) * 4;
    if ((rc = check_buf(gate, g, need_g, "gate"))) return rc;
    if ((rc = check_buf(up, g, need_u, "up"))) return rc;
    if ((rc = check_buf(out, g, static_cast<size_t>(rows) * cols * (out_f16 ? 2 : 4), "out"))) return rc;
    const size_t total = static_cast<size_t>(rows) * (cols / 4u);
    const uint32_t blocks = static_cast<uint32_t>(std::min<size_t>((total + 255) / 256, static_cast<size_t>(g->prop.multiProcessorCount) * 16u));
    const float* gp = static_cast<const float*>(gate->ptr) + gate_offset;
    const float* up_ = static_cast<const float*>(up->ptr) + up_offset;
    INJECT_LAUNCH();
    if (out_f16)
        silu_mul_kernel<uint16_t><<<blocks, 256, 0, g->stream>>>(rows, cols, gp, gate_pitch, up_, up_pitch, static_cast<uint16_t*>(out->ptr));
    else
        silu_mul_kernel<float><<<blocks, 256, 0, g->stream>>>(rows, cols, gp, gate_pitch, up_, up_pitch, static_cast<float*>(out->ptr));
    CUDA_TRY(cudaGetLastError());
    return LEXB_OK;
}

int lexb_prefill_chunks(uint32_t tokens, uint32_t limit, int gemm_ok, uint32_t* chunks, uint32_t max_chunks, uint32_t* count) {
    static const uint32_t GEMM_SIZES[6] = {512, 256, 128, 64, 32, 16};
    const uint32_t MAX_BATCH = 8;
    if (!count) return fail(LEXB_ERR_ARG, "lexb_prefill_chunks: null count");
    // prefill_limit: the largest GEMM size that is <= the wanted chunk (512 when 0), else MAX_BATCH
    uint32_t lim = MAX_BATCH;
    if (gemm_ok) {
        const uint32_t want = limit ? limit : 512u;
        for (uint32_t s : GEMM_SIZES)
            if (s <= want) { lim = s; break; }
    }
    uint32_t left = tokens, n = 0;
    while (left > 0) {
        uint32_t take = left < MAX_BATCH ? left : MAX_BATCH;
        if (gemm_ok)
            for (uint32_t s : GEMM_SIZES)
                if (s <= lim && s <= left) { take = s; break; }
        if (chunks) {
            if (n >= max_chunks) return fail(LEXB_ERR_ARG, "lexb_prefill_chunks: more than %u chunks", max_chunks);
            chunks[n] = take;
        }
        n++;
        left -= take;
    }
    *count = n;
    return LEXB_OK;
}

int lexb_debug_fail_next(int site, int nth, int cuda_error) {
    if (site < 0 || site >= SITE_COUNT) return fail(LEXB_ERR_ARG, "lexb_debug_fail_next: site %d outside [0, %d]", site, SITE_COUNT - 1);
    if (nth < 0 || cuda_error < 0) return fail(LEXB_ERR_ARG, "lexb_debug_fail_next: negative argument");
    std::lock_guard<std::mutex> lk(g_inject_lock);
    if (site == 0) {
        for (auto& in : g_inject) in = Injection{};
        return LEXB_OK;
    }
    g_inject[site].countdown = nth;
    g_inject[site].error = cuda_error ? cuda_error : static_cast<int>(cudaErrorUnknown);
    return LEXB_OK;
}

int lexb_shard_rows(uint32_t n, uint32_t world, uint32_t rank, uint32_t* n0, uint32_t* n1) {
    if (!n0 || !n1) return fail(LEXB_ERR_ARG, "lexb_shard_rows: null out");
    if (world == 0 || rank >= world) return fail(LEXB_ERR_ARG, "rank %u outside world %u", rank, world);
    if (n % 128u) return fail(LEXB_ERR_SHAPE, "sharding splits whole 128-row tiles; 128 does not divide n = %u", n);
    const uint32_t tiles = n / 128u, base = tiles / world, extra = tiles % world;
    const uint32_t first = rank * base + (rank < extra ? rank : extra);
    const uint32_t count = base + (rank < extra ? 1u : 0u);
    *n0 = first * 128u;
    *n1 = (first + count) * 128u;
    return LEXB_OK;
}

}  // extern "C"
