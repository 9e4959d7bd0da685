// Context, buffers, quantized-matrix upload / bit-exact dequantisation, the small decode operators and
// the synthetic-weight generator of the slai_b200 C ABI.
#include <stdarg.h>
#include <math.h>
#include <stdlib.h>

#include "common.cuh"
#include "gemv_frag.cuh"
#include "layout.cuh"
#include "dequant.cuh"

int slai_set_error(slai_ctx* ctx, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (ctx) ctx->last_error = buf;
    return code;
}

static thread_local std::string g_noctx_error;

// ------------------------------------------------------------------------------------------------
// context
// ------------------------------------------------------------------------------------------------
SLAI_API int slai_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

SLAI_API int slai_ctx_create(int device, slai_ctx** out) {
    if (!out) return SLAI_ERR_INVALID_ARG;
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        g_noctx_error = "no CUDA device available (this library has no CPU fallback)";
        return SLAI_ERR_CUDA;
    }
    if (device < 0 || device >= n) return SLAI_ERR_INVALID_ARG;
    slai_ctx* ctx = new slai_ctx();
    ctx->device = device;
    DeviceGuard guard(device);
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { delete ctx; return SLAI_ERR_CUDA; }
    if (prop.major != 10) {
        g_noctx_error = "slai_b200 is built for sm_100a only";
        delete ctx;
        return SLAI_ERR_CUDA;
    }
    ctx->sm_count = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreate(&ctx->ev0) != cudaSuccess || cudaEventCreate(&ctx->ev1) != cudaSuccess ||
        cudaMalloc(&ctx->d_counters, CNT_WORDS * sizeof(unsigned int)) != cudaSuccess ||
        cudaMemset(ctx->d_counters, 0, CNT_WORDS * sizeof(unsigned int)) != cudaSuccess) {
        delete ctx;
        return SLAI_ERR_CUDA;
    }
#ifdef SLAI_TRACE
    if (cudaMalloc(&ctx->trace_buf, (size_t)64 * TRACE_BLOCKS * TRACE_POINTS * 8) != cudaSuccess ||
        cudaMemset(ctx->trace_buf, 0, (size_t)64 * TRACE_BLOCKS * TRACE_POINTS * 8) != cudaSuccess ||
        cudaMalloc(&ctx->tl, ((size_t)TL_SLOTS * TL_CAP + 1) * 8) != cudaSuccess ||
        cudaMemset(ctx->tl, 0, ((size_t)TL_SLOTS * TL_CAP + 1) * 8) != cudaSuccess) {
        delete ctx;
        return SLAI_ERR_CUDA;
    }
#endif
    const char* pdl = getenv("SLAI_NO_PDL");
    ctx->use_pdl = !(pdl && pdl[0] == '1');
    *out = ctx;
    return SLAI_OK;
}

SLAI_API int slai_ctx_destroy(slai_ctx* ctx) {
    if (!ctx) return SLAI_OK;
    SLAI_ENTER(ctx);
    cudaStreamSynchronize(ctx->stream);
    for (auto& t : ctx->rope_tables) cudaFree(t.d_theta);
    if (ctx->d_scratch) cudaFree(ctx->d_scratch);
    for (void* p : ctx->retired_scratch) cudaFree(p);
    if (ctx->d_counters) cudaFree(ctx->d_counters);
    cudaEventDestroy(ctx->ev0);
    slai_tp_shutdown(ctx);
    cudaEventDestroy(ctx->ev1);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return SLAI_OK;
}

// After a synchronisation: did a bounded wait inside a kernel run out since the last check?
int slai_check_wait_flag(slai_ctx* ctx) {
    // Every wait inside the kernels (ring barriers, grid barrier, peer polls) is bounded; one that ran out raised this flag.
    unsigned int flag = 0;
    SLAI_CHECK_CUDA(ctx, cudaMemcpy(&flag, ctx->d_counters + CNT_ERR_FLAG, sizeof(flag), cudaMemcpyDeviceToHost));
    if (flag) {
        cudaMemset(ctx->d_counters + CNT_ERR_FLAG, 0, sizeof(flag));
        return slai_set_error(ctx, SLAI_ERR_TIMEOUT, "a bounded wait inside a kernel ran out (%s); results of the last launches are invalid",
                              flag == 1 ? "weight ring" : flag == 2 ? "grid barrier" : "tensor-parallel peer");
    }
    return SLAI_OK;
}
SLAI_API int slai_ctx_sync(slai_ctx* ctx) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return slai_check_wait_flag(ctx);
}
int slai_stats_mark(slai_ctx* ctx, int cls) {
    if (!ctx->stats_on) return SLAI_OK;
    cudaEvent_t e;
    SLAI_CHECK_CUDA(ctx, cudaEventCreate(&e));
    SLAI_CHECK_CUDA(ctx, cudaEventRecord(e, ctx->stream));
    ctx->stats_ev.push_back(e);
    ctx->stats_cls.push_back(cls);
    return SLAI_OK;
}

SLAI_API int slai_ctx_set_wait_limit(slai_ctx* ctx, uint32_t rounds) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    SLAI_REQUIRE(ctx, rounds >= 16, SLAI_ERR_INVALID_ARG, "wait limit of %u rounds is too short for a healthy launch", rounds);
    ctx->wait_limit = rounds;  // read when a launch is described: passes and graphs recorded earlier keep theirs
    return SLAI_OK;
}
SLAI_API const char* slai_last_error_string(slai_ctx* ctx) { return ctx ? ctx->last_error.c_str() : g_noctx_error.c_str(); }
SLAI_API void* slai_ctx_stream(slai_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }
SLAI_API int slai_ctx_device_info(slai_ctx* ctx, char* name, int name_len, int* sm_count) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    cudaDeviceProp prop;
    SLAI_CHECK_CUDA(ctx, cudaGetDeviceProperties(&prop, ctx->device));
    if (name && name_len > 0) snprintf(name, name_len, "%s", prop.name);
    if (sm_count) *sm_count = prop.multiProcessorCount;
    return SLAI_OK;
}

SLAI_API int slai_ctx_mem_info(slai_ctx* ctx, size_t* free_bytes, size_t* total_bytes) {
    if (!ctx || !free_bytes || !total_bytes) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_CHECK_CUDA(ctx, cudaMemGetInfo(free_bytes, total_bytes));
    return SLAI_OK;
}

SLAI_API int slai_malloc(slai_ctx* ctx, size_t bytes, void** d_out) {
    if (!ctx || !d_out) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    cudaError_t e = cudaMalloc(d_out, bytes ? bytes : 16);
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        return slai_set_error(ctx, SLAI_ERR_OOM, "out of device memory allocating %zu bytes", bytes);
    }
    SLAI_CHECK_CUDA(ctx, e);
    return SLAI_OK;
}
SLAI_API int slai_free(slai_ctx* ctx, void* d_ptr) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    SLAI_CHECK_CUDA(ctx, cudaFree(d_ptr));
    return SLAI_OK;
}
SLAI_API int slai_memset(slai_ctx* ctx, void* d_ptr, int value, size_t bytes) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_CHECK_CUDA(ctx, cudaMemsetAsync(d_ptr, value, bytes, ctx->stream));
    return SLAI_OK;
}
SLAI_API int slai_write_buffer(slai_ctx* ctx, void* d_dst, const void* h_src, size_t bytes) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return SLAI_OK;
}
SLAI_API int slai_read_buffer(slai_ctx* ctx, void* h_dst, const void* d_src, size_t bytes) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    SLAI_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return SLAI_OK;
}
SLAI_API int slai_malloc_host(slai_ctx* ctx, size_t bytes, void** h_out) {
    if (!ctx || !h_out) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_CHECK_CUDA(ctx, cudaMallocHost(h_out, bytes ? bytes : 16));
    return SLAI_OK;
}
SLAI_API int slai_free_host(slai_ctx* ctx, void* h_ptr) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_CHECK_CUDA(ctx, cudaFreeHost(h_ptr));
    return SLAI_OK;
}
// ---- recorded passes ---------------------------------------------------------------------------------
struct slai_pass {
    cudaGraphExec_t exec = nullptr;
};
SLAI_API int slai_pass_begin(slai_ctx* ctx) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_CHECK_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    return SLAI_OK;
}
SLAI_API int slai_pass_end(slai_ctx* ctx, slai_pass** out) {
    if (!ctx || !out) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    *out = nullptr;
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    if (e != cudaSuccess || !graph) {
        cudaGetLastError();
        return slai_set_error(ctx, SLAI_ERR_CUDA, "pass: recording failed (%s); a recorded call allocated or blocked",
                              cudaGetErrorString(e));
    }
    slai_pass* p = new slai_pass();
    e = cudaGraphInstantiate(&p->exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) {
        delete p;
        cudaGetLastError();
        return slai_set_error(ctx, SLAI_ERR_CUDA, "pass: %s", cudaGetErrorString(e));
    }
    *out = p;
    return SLAI_OK;
}
SLAI_API int slai_pass_launch(slai_ctx* ctx, slai_pass* pass, int times) {
    if (!ctx || !pass || !pass->exec || times < 0) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    for (int i = 0; i < times; i++) SLAI_CHECK_CUDA(ctx, cudaGraphLaunch(pass->exec, ctx->stream));
    return SLAI_OK;
}
SLAI_API int slai_pass_destroy(slai_ctx* ctx, slai_pass* pass) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    if (pass) {
        cudaStreamSynchronize(ctx->stream);
        if (pass->exec) cudaGraphExecDestroy(pass->exec);
        delete pass;
    }
    return SLAI_OK;
}

SLAI_API int slai_timer_start(slai_ctx* ctx) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_CHECK_CUDA(ctx, cudaEventRecord(ctx->ev0, ctx->stream));
    return SLAI_OK;
}
SLAI_API int slai_timer_stop(slai_ctx* ctx, float* ms) {
    if (!ctx || !ms) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_CHECK_CUDA(ctx, cudaEventRecord(ctx->ev1, ctx->stream));
    SLAI_CHECK_CUDA(ctx, cudaEventSynchronize(ctx->ev1));
    SLAI_CHECK_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev0, ctx->ev1));
    return SLAI_OK;
}

// ------------------------------------------------------------------------------------------------
// quantized matrices
// ------------------------------------------------------------------------------------------------
namespace {

__global__ void place_kernel(int fmt, const uint8_t* __restrict__ raw, uint8_t* __restrict__ dst, long long nrows, long long nbk,
                             long long K, int bb) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nrows * nbk) return;
    layout::place_block(fmt, raw + (size_t)i * bb, dst, i / nbk, i % nbk, K);
}

__global__ void dequant_kernel(int fmt, const uint8_t* __restrict__ data, long long row0, long long nrows, long long K,
                               float* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nrows * K) return;
    const long long r = row0 + i / K, k = i % K;
    out[i] = fmt == SLAI_FMT_F32 ? reinterpret_cast<const float*>(data)[r * K + k] : dequant_elem(fmt, data, K, r, k);
}

// Legacy blocks (quantization.rs:47-199) at upload: Q4_0 / Q5_0 -> the same values as Q8_0 blocks; Q4_1 / Q5_1 / Q8_K -> f32.
__device__ __forceinline__ int legacy_quant(int fmt, const uint8_t* b, int e) {  // element e (0..31) of a 32-element legacy block
    const int j = e & 15, hi = e >> 4;
    const int hdr = fmt == SLAI_FMT_Q4_0 ? 2 : fmt == SLAI_FMT_Q4_1 ? 4 : fmt == SLAI_FMT_Q5_0 ? 6 : 8;
    int q = hi ? (b[hdr + j] >> 4) : (b[hdr + j] & 0x0F);
    if (fmt == SLAI_FMT_Q5_0 || fmt == SLAI_FMT_Q5_1) {
        const uint8_t* h = b + hdr - 4;
        const uint32_t qh = (uint32_t)h[0] | ((uint32_t)h[1] << 8) | ((uint32_t)h[2] << 16) | ((uint32_t)h[3] << 24);
        q |= hi ? (int)((qh >> (j + 12)) & 0x10) : (int)(((qh >> j) << 4) & 0x10);
    }
    return q;
}
__global__ void legacy_to_q8_0_kernel(int fmt, const uint8_t* __restrict__ raw, uint8_t* __restrict__ out, long long nblocks, int bb) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nblocks * 32) return;
    const long long blk = i >> 5;
    const int e = (int)(i & 31);
    const uint8_t* b = raw + blk * bb;
    uint8_t* o = out + blk * 34;
    if (e < 2) o[e] = b[e];  // the f16 scale
    o[2 + e] = (uint8_t)(signed char)(legacy_quant(fmt, b, e) - (fmt == SLAI_FMT_Q4_0 ? 8 : 16));
}
__global__ void legacy_to_f32_kernel(int fmt, const uint8_t* __restrict__ raw, float* __restrict__ out, long long n, int be, int bb) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint8_t* b = raw + (i / be) * bb;
    const int e = (int)(i % be);
    if (fmt == SLAI_FMT_Q8_K) {
        float d;
        memcpy(&d, b, 4);
        out[i] = __fmul_rn(d, (float)(signed char)b[4 + e]);
        return;
    }
    const float d = dev_h2f(b[0] | (b[1] << 8)), m = dev_h2f(b[2] | (b[3] << 8));
    out[i] = __fadd_rn(__fmul_rn((float)legacy_quant(fmt, b, e), d), m);  // Q4_1 / Q5_1: q * d + m
}

}  // namespace

static int qmatrix_alloc(slai_ctx* ctx, int fmt, int64_t nrows, int64_t ncols, size_t nbytes, slai_qmatrix** out) {
    SLAI_REQUIRE(ctx, out, SLAI_ERR_INVALID_ARG, "qmatrix: null output");
    *out = nullptr;
    const int be = fmt_block_elems(fmt), bb = fmt_block_bytes(fmt);
    SLAI_REQUIRE(ctx, be > 0, SLAI_ERR_UNSUPPORTED_FORMAT,
                 "qmatrix: GGML type %d is not supported (supported: F32, Q8_0, Q4_K, Q5_K, Q6_K and the legacy Q4_0, Q4_1, Q5_0, Q5_1, Q8_K)", fmt);
    SLAI_REQUIRE(ctx, nrows > 0 && ncols > 0 && ncols % be == 0, SLAI_ERR_SHAPE,
                 "qmatrix: %lld x %lld is not a whole number of %d-element blocks per row", (long long)nrows,
                 (long long)ncols, be);
    SLAI_REQUIRE(ctx, fmt == SLAI_FMT_F32 || ncols % 4 == 0, SLAI_ERR_SHAPE, "qmatrix: ncols must be a multiple of 4");
    SLAI_REQUIRE(ctx, nrows < (1ll << 31) && ncols < (1ll << 31), SLAI_ERR_SHAPE, "qmatrix: dimension too large");
    SLAI_REQUIRE(ctx, nbytes == (size_t)nrows * (ncols / be) * bb, SLAI_ERR_SHAPE,
                 "qmatrix: expected %zu bytes of blocks, got %zu", (size_t)nrows * (ncols / be) * bb, nbytes);
    slai_qmatrix* m = new slai_qmatrix();
    m->ctx = ctx; m->src_fmt = fmt; m->fmt = legacy_device_format(fmt); m->nrows = nrows; m->ncols = ncols;
    m->tile_bytes = m->fmt == SLAI_FMT_F32 ? ncols * 4 : layout::tile_bytes(m->fmt, ncols);
    m->bytes = (size_t)layout::matrix_bytes(m->fmt, nrows, ncols);
    cudaError_t e = cudaMalloc(&m->data, m->bytes + 256);
    if (e != cudaSuccess) {
        cudaGetLastError();
        delete m;
        return slai_set_error(ctx, SLAI_ERR_OOM, "qmatrix: cannot allocate %zu bytes", m->bytes);
    }
    *out = m;
    return SLAI_OK;
}

SLAI_API int slai_qmatrix_create_from_device(slai_ctx* ctx, int fmt, int64_t nrows, int64_t ncols, const void* d_blocks,
                                             size_t nbytes, slai_qmatrix** out) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    int rc = qmatrix_alloc(ctx, fmt, nrows, ncols, nbytes, out);
    if (rc) return rc;
    slai_qmatrix* m = *out;
    const int be = fmt_block_elems(fmt), bb = fmt_block_bytes(fmt);
    const long long nbk = ncols / be;
    if (fmt == SLAI_FMT_F32) {
        SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(m->data, d_blocks, nbytes, cudaMemcpyDeviceToDevice, ctx->stream));
    } else if (m->fmt != fmt && m->fmt == SLAI_FMT_F32) {  // Q4_1 / Q5_1 / Q8_K: dense f32
        const long long n = nrows * ncols;
        legacy_to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(fmt, (const uint8_t*)d_blocks, (float*)m->data, n, be, bb);
        SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    } else if (m->fmt != fmt) {  // Q4_0 / Q5_0: the same values as Q8_0 blocks, then the usual placement
        const long long total = nrows * nbk;
        uint8_t* q8 = nullptr;
        SLAI_CHECK_CUDA(ctx, cudaMalloc(&q8, (size_t)total * 34));
        legacy_to_q8_0_kernel<<<(unsigned)((total * 32 + 255) / 256), 256, 0, ctx->stream>>>(fmt, (const uint8_t*)d_blocks, q8, total, bb);
        SLAI_CHECK_CUDA(ctx, cudaMemsetAsync(m->data, 0, m->bytes, ctx->stream));
        place_kernel<<<(unsigned)((total + 127) / 128), 128, 0, ctx->stream>>>(SLAI_FMT_Q8_0, q8, m->data, nrows, nbk, ncols, 34);
        cudaError_t e = cudaGetLastError();
        cudaStreamSynchronize(ctx->stream);
        cudaFree(q8);
        SLAI_CHECK_CUDA(ctx, e);
    } else {
        SLAI_CHECK_CUDA(ctx, cudaMemsetAsync(m->data, 0, m->bytes, ctx->stream));  // padding rows / steps are zero
        const long long total = nrows * nbk;
        place_kernel<<<(unsigned)((total + 127) / 128), 128, 0, ctx->stream>>>(fmt, (const uint8_t*)d_blocks, m->data, nrows, nbk, ncols, bb);
        SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    }
    return SLAI_OK;
}

SLAI_API int slai_qmatrix_create(slai_ctx* ctx, int fmt, int64_t nrows, int64_t ncols, const void* h_blocks, size_t nbytes,
                                 slai_qmatrix** out) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_REQUIRE(ctx, h_blocks, SLAI_ERR_INVALID_ARG, "qmatrix: null block pointer");
    void* tmp = nullptr;
    cudaError_t e = cudaMalloc(&tmp, nbytes ? nbytes : 16);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return slai_set_error(ctx, SLAI_ERR_OOM, "qmatrix: cannot allocate %zu bytes of staging", nbytes);
    }
    int rc = SLAI_OK;
    if (cudaMemcpyAsync(tmp, h_blocks, nbytes, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess)
        rc = slai_set_error(ctx, SLAI_ERR_CUDA, "qmatrix: upload failed");
    if (!rc) rc = slai_qmatrix_create_from_device(ctx, fmt, nrows, ncols, tmp, nbytes, out);
    cudaStreamSynchronize(ctx->stream);
    cudaFree(tmp);
    return rc;
}

SLAI_API int slai_qmatrix_destroy(slai_qmatrix* m) {
    if (!m) return SLAI_OK;
    SLAI_ENTER(m->ctx);
    if (m->owns && m->data) {
        cudaStreamSynchronize(m->ctx->stream);
        cudaFree(m->data);
    }
    delete m;
    return SLAI_OK;
}
SLAI_API int slai_qmatrix_shape(const slai_qmatrix* m, int* fmt, int64_t* nrows, int64_t* ncols) {
    if (!m) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    if (fmt) *fmt = m->src_fmt;
    if (nrows) *nrows = m->nrows;
    if (ncols) *ncols = m->ncols;
    return SLAI_OK;
}
SLAI_API size_t slai_qmatrix_device_bytes(const slai_qmatrix* m) { return m ? m->bytes : 0; }

SLAI_API int slai_qmatrix_dequantize(slai_ctx* ctx, const slai_qmatrix* m, float* d_out) {
    if (!ctx || !m || !d_out) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    const long long total = m->nrows * m->ncols;
    dequant_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(m->fmt, m->data, 0, m->nrows, m->ncols, d_out);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
SLAI_API int slai_qmatrix_dequantize_row(slai_ctx* ctx, const slai_qmatrix* m, int64_t row, float* d_out) {
    if (!ctx || !m || !d_out) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_REQUIRE(ctx, row >= 0 && row < m->nrows, SLAI_ERR_INVALID_ARG, "dequantize_row: row %lld out of range", (long long)row);
    dequant_kernel<<<(unsigned)((m->ncols + 255) / 256), 256, 0, ctx->stream>>>(m->fmt, m->data, row, 1, m->ncols, d_out);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}

SLAI_API int slai_gemv_quant(slai_ctx* ctx, float* d_out, const slai_qmatrix* w, const float* d_v, int n_batch) {
    if (!ctx || !w || !d_out || !d_v) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_REQUIRE(ctx, n_batch >= 1 && n_batch <= 8, SLAI_ERR_INVALID_ARG, "gemv: n_batch=%d must be in 1..8", n_batch);
    // A batch streams a quantised matrix once (gemv_batch.cu); dense f32 matrices take the vectors one by one.
    if (n_batch > 1 && gemv_batch_supported(w)) return gemv_batch_launch(ctx, d_out, w, d_v, n_batch);
    for (int b = 0; b < n_batch; b++) {
        GemvLaunch L;
        L.fmt = w->fmt;
        L.K = (int)w->ncols;
        L.nseg = 1;
        L.seg[0].w = w->data;
        L.seg[0].tile_bytes = w->tile_bytes;
        L.seg[0].rows = (int)w->nrows;
        L.v = d_v + (size_t)b * w->ncols;
        L.out = d_out + (size_t)b * w->nrows;
        int rc = gemv_launch(ctx, L);
        if (rc) return rc;
    }
    return SLAI_OK;
}

// hb = silu(Wgate n(x)) * (Wup n(x)), n = RmsNorm with `d_norm_w` (null: no normalisation): the feed-forward front half
// of a Llama layer in one kernel, both matrices streamed tile by tile side by side.
SLAI_API int slai_ffn_gate_up(slai_ctx* ctx, float* d_out, const slai_qmatrix* w_gate, const slai_qmatrix* w_up, const float* d_x,
                              const float* d_norm_w, float eps) {
    if (!ctx || !w_gate || !w_up || !d_out || !d_x) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_REQUIRE(ctx, w_gate->fmt == w_up->fmt && w_gate->fmt != SLAI_FMT_F32, SLAI_ERR_UNSUPPORTED_FORMAT,
                 "ffn_gate_up: both matrices must have the same quantised format");
    SLAI_REQUIRE(ctx, w_gate->nrows == w_up->nrows && w_gate->ncols == w_up->ncols, SLAI_ERR_SHAPE, "ffn_gate_up: gate is %lldx%lld, up is %lldx%lld",
                 (long long)w_gate->nrows, (long long)w_gate->ncols, (long long)w_up->nrows, (long long)w_up->ncols);
    GemvLaunch L;
    L.fmt = w_gate->fmt;
    L.K = (int)w_gate->ncols;
    L.nseg = 2;
    for (int i = 0; i < 2; i++) {
        const slai_qmatrix* w = i == 0 ? w_gate : w_up;
        L.seg[i].w = w->data;
        L.seg[i].tile_bytes = w->tile_bytes;
        L.seg[i].rows = (int)w->nrows;
    }
    L.v = d_x;
    L.out = d_out;
    L.pro = d_norm_w ? PRO_RMS : PRO_NONE;
    L.norm_w = d_norm_w;
    L.eps = eps;
    L.epi = EPI_SILU;
    return gemv_launch(ctx, L);
}

// ------------------------------------------------------------------------------------------------
// small operators
// ------------------------------------------------------------------------------------------------
namespace {

constexpr int NT = 256;

__device__ __forceinline__ float blk_sum(float x, float* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = x;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) t += sh[w];
    return t;
}
__device__ __forceinline__ float blk_max(float x, float* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = x;
    __syncthreads();
    float t = -INFINITY;
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) t = fmaxf(t, sh[w]);
    return t;
}

// One block per row of n elements (a single vector: one block).
__global__ void rms_norm_kernel(float* out, const float* x, const float* w, long long n, float eps) {
    __shared__ float sh[32];
    out += (size_t)blockIdx.x * n;
    x += (size_t)blockIdx.x * n;
    float ss = 0.f;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) ss += x[i] * x[i];
    ss = blk_sum(ss, sh);
    const float rms = 1.0f / sqrtf(ss / (float)n + eps);
    for (long long i = threadIdx.x; i < n; i += blockDim.x) out[i] = (x[i] * rms) * w[i];
}

__global__ void layernorm_kernel(float* out, const float* x, long long n, float eps, const float* gamma, const float* beta) {
    __shared__ float sh[32];
    float s = 0.f;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
    const float mean = blk_sum(s, sh) / (float)n;
    float ss = 0.f;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) {
        const float d = x[i] - mean;
        ss += d * d;
    }
    const float var = blk_sum(ss, sh) / (float)n;
    const float scale = 1.0f / sqrtf(var + eps);
    for (long long i = threadIdx.x; i < n; i += blockDim.x) {
        float y = (x[i] - mean) * scale;
        if (gamma) y *= gamma[i];
        if (beta) y += beta[i];
        out[i] = y;
    }
}

__global__ void softmax_cols_kernel(float* m, long long nrows, long long col_stride) {
    __shared__ float sh[32];
    float* col = m + (size_t)blockIdx.x * col_stride;
    float mx = -INFINITY;
    for (long long i = threadIdx.x; i < nrows; i += blockDim.x) mx = fmaxf(mx, col[i]);
    mx = blk_max(mx, sh);
    float s = 0.f;
    for (long long i = threadIdx.x; i < nrows; i += blockDim.x) {
        const float e = expf(col[i] - mx);
        col[i] = e;
        s += e;
    }
    s = blk_sum(s, sh);
    for (long long i = threadIdx.x; i < nrows; i += blockDim.x) col[i] = col[i] / s;
}

__global__ void silu_gate_kernel(float* h1, const float* h2, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float x = h1[i];
        h1[i] = h2[i] * (x / (1.0f + expf(-x)));
    }
}

__device__ float unary_eval(int op, float x, float a0, float a1) {
    switch (op) {
        case 0: return fabsf(x);
        case 1: return isnan(x) ? x : copysignf(1.0f, x);
        case 2: return -x;
        case 3: return x > 0.f ? 1.f : 0.f;
        case 4: return x > 0.f ? x : expf(x) - 1.0f;
        case 5: {
            const float A = 0.044715f, S = 0.7978846f;
            return 0.5f * x * (1.0f + tanhf(S * x * (1.0f + A * x * x)));
        }
        case 6: return x * (1.0f / (1.0f + expf(-1.702f * x)));
        case 7: return x / (1.0f + expf(-x));
        case 8: return tanhf(x);
        case 9: return sinf(x);
        case 10: return cosf(x);
        case 11: return fmaxf(x, 0.f);
        case 12: return 1.0f / (1.0f + expf(-x));
        case 13: return fminf(1.0f, fmaxf(0.0f, (x + 3.0f) / 6.0f));
        case 14: return x * x;
        case 15: return sqrtf(x);
        case 16: return logf(x);
        case 17: return fmaxf(x, 0.f) + fminf(x, 0.f) * a0;
        case 18: return fminf(fmaxf(x, a0), a1);
        case 19: return x * a0;
        case 20: return x + a0;
    }
    return NAN;
}
__global__ void unary_kernel(int op, float* dst, const float* src, long long n, float a0, float a1) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = unary_eval(op, src[i], a0, a1);
}

// mode 0: a += b, 1: a *= b, 2: a = b
__global__ void binary_kernel(int mode, float* a, const float* b, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] = mode == 0 ? a[i] + b[i] : mode == 1 ? a[i] * b[i] : b[i];
}

__global__ void rope_kernel(int neox, float* q, long long q_len, float* k, int head_size, int kv_dim, int pos,
                            const float* theta) {
    const long long pair = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long i = 2 * pair;
    if (i >= q_len) return;
    const int hd = (int)(i % head_size);
    const float ang = (float)pos * theta[hd >> 1];
    float sn, cs;
    sincosf(ang, &sn, &cs);
    long long i0, i1;
    if (!neox) {
        i0 = i;
        i1 = i + 1;
    } else {
        const long long head = i / head_size;
        i0 = pair + head * head_size / 2;
        i1 = i0 + head_size / 2;
    }
    const float q0 = q[i0], q1 = q[i1];
    q[i0] = cs * q0 - sn * q1;
    q[i1] = sn * q0 + cs * q1;
    if (i < kv_dim) {
        const float k0 = k[i0], k1 = k[i1];
        k[i0] = cs * k0 - sn * k1;
        k[i1] = sn * k0 + cs * k1;
    }
}

__global__ void set_int_kernel(int* dst, int value) { *dst = value; }

template <typename T>
__global__ void kv_append_kernel(T* kc, T* vc, const float* k, const float* v, int kv_dim, long long off) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < kv_dim) {
        kc[off + i] = (T)k[i];
        vc[off + i] = (T)v[i];
    }
}
template <>
__global__ void kv_append_kernel<__half>(__half* kc, __half* vc, const float* k, const float* v, int kv_dim, long long off) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < kv_dim) {
        kc[off + i] = __float2half_rn(k[i]);
        vc[off + i] = __float2half_rn(v[i]);
    }
}

// first maximal index (nalgebra `imax`): ties resolve to the smaller index.  ARG_BLOCKS blocks scan a slice each;
// the last one to finish (ticket) combines the per-block results.
constexpr int ARG_BLOCKS = 32, ARG_THREADS = 256;
__device__ __forceinline__ bool arg_better(float a, int ai, float b, int bi) { return a > b || (a == b && ai < bi); }
__global__ void __launch_bounds__(ARG_THREADS) argmax_kernel(const float* v, long long n, int* out, unsigned int* work /* ticket, then ARG_BLOCKS x (value, index) */) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float sv[ARG_THREADS / 32];
    __shared__ int si[ARG_THREADS / 32];
    __shared__ int s_last;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    const long long per = (n + ARG_BLOCKS - 1) / ARG_BLOCKS;
    const long long lo = per * blockIdx.x, hi = lo + per < n ? lo + per : n;
    for (long long i = lo + threadIdx.x; i < hi; i += ARG_THREADS) {
        const float x = v[i];
        if (arg_better(x, (int)i, best, bi)) {
            best = x;
            bi = (int)i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (arg_better(ob, oi, best, bi)) {
            best = ob;
            bi = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = best;
        si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < ARG_THREADS / 32; w++)
            if (arg_better(sv[w], si[w], best, bi)) {
                best = sv[w];
                bi = si[w];
            }
        work[1 + 2 * blockIdx.x] = __float_as_uint(best);
        work[2 + 2 * blockIdx.x] = (unsigned int)bi;
        __threadfence();
        const unsigned int t = atomicAdd(work, 1u);
        s_last = t == gridDim.x - 1;
        if (s_last) {
            *work = 0;
            __threadfence();
            for (int b = 0; b < (int)gridDim.x; b++) {
                const float ob = __uint_as_float(__ldcg(work + 1 + 2 * b));
                const int oi = (int)__ldcg(work + 2 + 2 * b);
                if (arg_better(ob, oi, best, bi)) {
                    best = ob;
                    bi = oi;
                }
            }
            *out = bi == 0x7fffffff ? 0 : bi;
        }
    }
}

// cos / sin of the token's RoPE angles, once per token (the q/k/v kernels of all layers read the pairs instead of
// evaluating sincosf in their epilogues)
__device__ __forceinline__ void rope_pairs(const float* theta, float* cs, int half, const int* d_pos) {
    if (cs && blockIdx.x == 0 && (int)threadIdx.x < half) {
        float sn, c;
        sincosf((float)(*d_pos) * theta[threadIdx.x], &sn, &c);
        cs[2 * threadIdx.x] = c;
        cs[2 * threadIdx.x + 1] = sn;
    }
}
__global__ void embed_f32_kernel(float* x, const float* table, int dim, const int* d_token, const float* wpe, const int* d_pos,
                                 const float* theta, float* cs, int half) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    rope_pairs(theta, cs, half, d_pos);
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= dim) return;
    float y = table[(size_t)(*d_token) * dim + i];
    if (wpe) y += wpe[(size_t)(*d_pos) * dim + i];
    x[i] = y;
}
__global__ void embed_q_kernel(float* x, int fmt, const uint8_t* data, int dim, const int* d_token, const float* wpe,
                               const int* d_pos, const float* theta, float* cs, int half) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    rope_pairs(theta, cs, half, d_pos);
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= dim) return;
    const long long row = *d_token;
    float y = fmt == SLAI_FMT_F32 ? reinterpret_cast<const float*>(data)[row * dim + i] : dequant_elem(fmt, data, dim, row, i);
    if (wpe) y += wpe[(size_t)(*d_pos) * dim + i];
    x[i] = y;
}
// Advance the device-side loop state without a host round trip: pos <- pos + 1, step <- step + 1 and
//   greedy (d_next != NULL): token <- *d_next, history[step] <- *d_next
//   forced (d_next == NULL): token <- history[step]   (prompt processing)
__global__ void advance_kernel(int* d_token, int* d_pos, const int* d_next, int* d_history, int* d_step, int vocab) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int step = *d_step;
    int nx;
    if (d_next) {
        nx = *d_next;
        d_history[step] = nx;
    } else {
        nx = d_history[step];
    }
    nx = nx < 0 ? 0 : (nx >= vocab ? vocab - 1 : nx);  // whatever a kernel produced, the embedding lookup stays inside its table
    *d_token = nx;
    *d_pos = *d_pos + 1;
    *d_step = step + 1;
}

template <typename... Args>
int launch_pdl(slai_ctx* ctx, void (*kern)(Args...), dim3 grid, dim3 block, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    SLAI_CHECK_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, args...));
    return SLAI_OK;
}

}  // namespace

SLAI_API int slai_rms_norm(slai_ctx* ctx, float* d_out, const float* d_x, const float* d_w, int64_t n, float eps) {
    if (!ctx || !d_out || !d_x || !d_w || n <= 0) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    rms_norm_kernel<<<1, 1024, 0, ctx->stream>>>(d_out, d_x, d_w, n, eps);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
// RmsNorm of `rows` vectors of n elements with the same weights.
int rms_norm_rows_launch(slai_ctx* ctx, float* d_out, const float* d_x, const float* d_w, int64_t n, int rows, float eps) {
    rms_norm_kernel<<<rows, 1024, 0, ctx->stream>>>(d_out, d_x, d_w, n, eps);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
SLAI_API int slai_layernorm(slai_ctx* ctx, float* d_out, const float* d_x, int64_t n, float eps, const float* d_gamma,
                            const float* d_beta) {
    if (!ctx || !d_out || !d_x || n <= 0) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    layernorm_kernel<<<1, 1024, 0, ctx->stream>>>(d_out, d_x, n, eps, d_gamma, d_beta);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
SLAI_API int slai_softmax_cols(slai_ctx* ctx, float* d_m, int64_t nrows, int64_t ncols, int64_t col_stride) {
    if (!ctx || !d_m || nrows <= 0 || ncols <= 0) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_REQUIRE(ctx, col_stride >= nrows, SLAI_ERR_SHAPE, "softmax: col_stride < nrows");
    softmax_cols_kernel<<<(unsigned)ncols, NT, 0, ctx->stream>>>(d_m, nrows, col_stride);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
SLAI_API int slai_silu_gate(slai_ctx* ctx, float* d_h1, const float* d_h2, int64_t n) {
    if (!ctx || !d_h1 || !d_h2 || n <= 0) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    silu_gate_kernel<<<(unsigned)((n + NT - 1) / NT), NT, 0, ctx->stream>>>(d_h1, d_h2, n);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
SLAI_API int slai_unary(slai_ctx* ctx, int op, float* d_dst, const float* d_src, int64_t n, const float args4[4]) {
    if (!ctx || !d_dst || !d_src || n <= 0) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_REQUIRE(ctx, op >= 0 && op <= 20, SLAI_ERR_INVALID_ARG, "unary: unknown op %d", op);
    const float a0 = args4 ? args4[0] : 0.f, a1 = args4 ? args4[1] : 0.f;
    long long blocks = (n + NT - 1) / NT;
    if (blocks > 65535) blocks = 65535;  // launch_capped: grid-stride above the cap (ops/unary.rs:222)
    unary_kernel<<<(unsigned)blocks, NT, 0, ctx->stream>>>(op, d_dst, d_src, n, a0, a1);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
static int binary(slai_ctx* ctx, int mode, float* a, const float* b, int64_t n) {
    if (!ctx || !a || !b || n <= 0) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    binary_kernel<<<(unsigned)((n + NT - 1) / NT), NT, 0, ctx->stream>>>(mode, a, b, n);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
SLAI_API int slai_add_assign(slai_ctx* ctx, float* d_a, const float* d_b, int64_t n) { return binary(ctx, 0, d_a, d_b, n); }
SLAI_API int slai_mul_assign(slai_ctx* ctx, float* d_a, const float* d_b, int64_t n) { return binary(ctx, 1, d_a, d_b, n); }
SLAI_API int slai_copy(slai_ctx* ctx, float* d_dst, const float* d_src, int64_t n) { return binary(ctx, 2, d_dst, d_src, n); }

const float* rope_table(slai_ctx* ctx, int head_size, float base) {
    for (auto& t : ctx->rope_tables)
        if (t.head_size == head_size && t.base == base) return t.d_theta;
    // theta_i = base^(-(2i)/head_size), evaluated with the host libm like the CPU twin
    // (models/llama2/cpu.rs:468: `10000.0_f32.powf(-head_dim / head_size as f32)`).
    std::vector<float> th(head_size / 2);
    for (int i = 0; i < head_size / 2; i++) th[i] = powf(base, -(float)(2 * i) / (float)head_size);
    RopeTable t;
    t.head_size = head_size;
    t.base = base;
    t.d_theta = nullptr;
    if (cudaMalloc(&t.d_theta, sizeof(float) * (head_size / 2 + 4)) != cudaSuccess) return nullptr;
    if (cudaMemcpy(t.d_theta, th.data(), sizeof(float) * (head_size / 2), cudaMemcpyHostToDevice) != cudaSuccess) return nullptr;
    ctx->rope_tables.push_back(t);
    return t.d_theta;
}

SLAI_API int slai_rope(slai_ctx* ctx, int variant, float* d_q, int64_t q_len, float* d_k, int head_size, int kv_dim, int pos,
                       float base_freq) {
    if (!ctx || !d_q || !d_k) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    // the reference asserts even lengths and len(q) >= len(k) (ops/rope.rs:58-63)
    SLAI_REQUIRE(ctx, q_len > 0 && q_len % 2 == 0 && kv_dim % 2 == 0 && kv_dim <= q_len, SLAI_ERR_SHAPE,
                 "rope: q_len=%lld and kv_dim=%d must be even with kv_dim <= q_len", (long long)q_len, kv_dim);
    SLAI_REQUIRE(ctx, head_size > 0 && head_size % 2 == 0 && q_len % head_size == 0, SLAI_ERR_SHAPE,
                 "rope: head_size=%d must be even and divide q_len", head_size);
    SLAI_REQUIRE(ctx, variant == 0 || variant == 1, SLAI_ERR_INVALID_ARG, "rope: unknown variant %d", variant);
    const float* th = rope_table(ctx, head_size, base_freq);
    SLAI_REQUIRE(ctx, th, SLAI_ERR_CUDA, "rope: cannot build the frequency table");
    const long long pairs = q_len / 2;
    rope_kernel<<<(unsigned)((pairs + NT - 1) / NT), NT, 0, ctx->stream>>>(variant, d_q, q_len, d_k, head_size, kv_dim, pos, th);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}

SLAI_API int slai_kv_append(slai_ctx* ctx, void* d_key_cache, void* d_value_cache, int kv_dtype, const float* d_k,
                            const float* d_v, int kv_dim, int pos) {
    if (!ctx || !d_key_cache || !d_value_cache || !d_k || !d_v || kv_dim <= 0 || pos < 0) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    const long long off = (long long)pos * kv_dim;
    const unsigned blocks = (kv_dim + NT - 1) / NT;
    if (kv_dtype == SLAI_KV_F16)
        kv_append_kernel<__half><<<blocks, NT, 0, ctx->stream>>>((__half*)d_key_cache, (__half*)d_value_cache, d_k, d_v, kv_dim, off);
    else if (kv_dtype == SLAI_KV_F32)
        kv_append_kernel<float><<<blocks, NT, 0, ctx->stream>>>((float*)d_key_cache, (float*)d_value_cache, d_k, d_v, kv_dim, off);
    else
        return slai_set_error(ctx, SLAI_ERR_INVALID_ARG, "kv_append: unknown cache type %d", kv_dtype);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}

SLAI_API int slai_attention(slai_ctx* ctx, const slai_attn_params* p, const float* d_q, const void* d_key_cache,
                            const void* d_value_cache, int kv_dtype, float* d_xb) {
    if (!ctx || !p || !d_q || !d_key_cache || !d_value_cache || !d_xb) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_REQUIRE(ctx, p->pos < p->seq_len, SLAI_ERR_SHAPE, "attention: pos=%u >= seq_len=%u", p->pos, p->seq_len);
    SLAI_REQUIRE(ctx, p->kv_mul > 0 && p->n_heads % p->kv_mul == 0 && p->kv_dim == p->n_heads / p->kv_mul * p->head_size,
                 SLAI_ERR_SHAPE, "attention: inconsistent head counts");
    SLAI_REQUIRE(ctx, kv_dtype == SLAI_KV_F16 || kv_dtype == SLAI_KV_F32, SLAI_ERR_INVALID_ARG, "attention: unknown cache type");
    // position scalar on the device (the kernels read it from memory so that CUDA graphs can be replayed)
    // (written by a one-thread kernel that takes the value as an argument: a memcpy from this stack frame would leave a
    // dangling host pointer in a recorded pass)
    int* d_pos = reinterpret_cast<int*>(ctx->d_counters + CNT_ATTN_POS);
    const int pos = (int)p->pos;
    set_int_kernel<<<1, 1, 0, ctx->stream>>>(d_pos, pos);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    AttnLaunch A;
    A.q = d_q; A.kcache = d_key_cache; A.vcache = d_value_cache; A.kv_dtype = kv_dtype;
    A.pos_stride = p->kv_dim; A.head_stride = p->head_size;
    A.n_heads = (int)p->n_heads; A.kv_mul = (int)p->kv_mul; A.head_size = (int)p->head_size;
    A.d_pos = d_pos; A.max_pos = pos; A.out = d_xb; A.pdl = false; A.scratch = nullptr; A.scratch_bytes = 0;
    return attention_launch(ctx, A);
}

SLAI_API int slai_argmax(slai_ctx* ctx, const float* d_v, int64_t n, int32_t* d_index_out) {
    if (!ctx || !d_v || !d_index_out || n <= 0) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    return launch_argmax(ctx, d_v, n, d_index_out, false);
}

int launch_argmax(slai_ctx* ctx, const float* v, int64_t n, int32_t* d_out, bool pdl) {
    return launch_pdl(ctx, argmax_kernel, dim3(ARG_BLOCKS), dim3(ARG_THREADS), pdl, v, (long long)n, (int*)d_out, ctx->d_counters + CNT_ARGMAX);
}
int launch_embed_f32(slai_ctx* ctx, float* x, const float* table, int dim, const int* d_token, const float* wpe,
                     const int* d_pos, bool pdl, const float* rope_theta, float* rope_cs, int rope_half) {
    return launch_pdl(ctx, embed_f32_kernel, dim3((dim + NT - 1) / NT), dim3(NT), pdl, x, table, dim, d_token, wpe, d_pos, rope_theta,
                      rope_cs, rope_half);
}
int launch_embed_q8(slai_ctx* ctx, float* x, const slai_qmatrix* wte, const int* d_token, const float* wpe,
                    const int* d_pos, bool pdl, const float* rope_theta, float* rope_cs, int rope_half) {
    const int dim = (int)wte->ncols;
    return launch_pdl(ctx, embed_q_kernel, dim3((dim + NT - 1) / NT), dim3(NT), pdl, x, wte->fmt, (const uint8_t*)wte->data, dim,
                      d_token, wpe, d_pos, rope_theta, rope_cs, rope_half);
}
int launch_advance(slai_ctx* ctx, int* d_token, int* d_pos, const int32_t* d_next, int32_t* d_history, int vocab, bool pdl) {
    // d_history[-1] is not used; the step counter lives right after the position scalar (see models)
    return launch_pdl(ctx, advance_kernel, dim3(1), dim3(1), pdl, d_token, d_pos, (const int*)d_next, (int*)d_history,
                      d_pos + 1, vocab);
}

// ------------------------------------------------------------------------------------------------
// synthetic weights
// ------------------------------------------------------------------------------------------------
namespace {

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
// standard normal from a counter: Box-Muller on two 24-bit uniforms
__device__ __forceinline__ float normal_at(uint64_t seed, uint64_t idx) {
    const uint64_t h = splitmix64(seed ^ splitmix64(idx));
    const float u1 = ((float)((h >> 40) & 0xFFFFFF) + 1.0f) * (1.0f / 16777217.0f);
    const float u2 = (float)((h >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);
    return sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
}
__device__ __forceinline__ unsigned short f2h_bits(float x) { return __half_as_ushort(__float2half_rn(x)); }
__device__ __forceinline__ float sdiv(float a, float b) { return b != 0.f ? a / b : 0.f; }

__global__ void synth_normal_kernel(float* out, long long n, uint64_t seed, float std) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = normal_at(seed, (uint64_t)i) * std;
}

// one thread per block of 32 (Q8_0) or 256 (K-quants) values; simple min/max quantisers that always
// yield valid blocks (the reference has no quantiser; quality is irrelevant to parity)
__global__ void synth_blocks_kernel(int fmt, uint8_t* out, long long nblocks, uint64_t seed, float std) {
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    if (fmt == SLAI_FMT_Q8_0) {
        float x[32];
        float amax = 0.f;
        for (int i = 0; i < 32; i++) {
            x[i] = normal_at(seed, (uint64_t)b * 32 + i) * std;
            amax = fmaxf(amax, fabsf(x[i]));
        }
        const unsigned short sb = f2h_bits(amax / 127.0f);
        const float sv = __half2float(__ushort_as_half(sb));
        uint8_t* o = out + b * 34;
        o[0] = sb & 0xFF;
        o[1] = sb >> 8;
        for (int i = 0; i < 32; i++) {
            int q = (int)rintf(sdiv(x[i], sv));
            q = max(-127, min(127, q));
            o[2 + i] = (uint8_t)(signed char)q;
        }
        return;
    }
    float x[256];
    for (int i = 0; i < 256; i++) x[i] = normal_at(seed, (uint64_t)b * 256 + i) * std;
    if (fmt == SLAI_FMT_Q4_K || fmt == SLAI_FMT_Q5_K) {
        const int levels = fmt == SLAI_FMT_Q4_K ? 15 : 31;
        float s[8], o8[8], smax = 0.f, omax = 0.f;
        for (int j = 0; j < 8; j++) {
            float lo = 0.f, hi = -INFINITY;
            for (int i = 0; i < 32; i++) {
                lo = fminf(lo, x[32 * j + i]);
                hi = fmaxf(hi, x[32 * j + i]);
            }
            hi = fmaxf(hi, lo);
            s[j] = (hi - lo) / (float)levels;
            o8[j] = -lo;
            smax = fmaxf(smax, s[j]);
            omax = fmaxf(omax, o8[j]);
        }
        const unsigned short db = f2h_bits(smax / 63.0f), mb = f2h_bits(omax / 63.0f);
        const float dv = __half2float(__ushort_as_half(db)), mv = __half2float(__ushort_as_half(mb));
        uint8_t sc[8], mn[8];
        for (int j = 0; j < 8; j++) {
            sc[j] = (uint8_t)max(0, min(63, (int)rintf(sdiv(s[j], dv))));
            mn[j] = (uint8_t)max(0, min(63, (int)rintf(sdiv(o8[j], mv))));
        }
        const int bb = fmt == SLAI_FMT_Q4_K ? 144 : 176;
        uint8_t* o = out + b * bb;
        o[0] = db & 0xFF; o[1] = db >> 8; o[2] = mb & 0xFF; o[3] = mb >> 8;
        for (int j = 0; j < 4; j++) {
            o[4 + j] = sc[j] | ((sc[j + 4] >> 4) << 6);
            o[8 + j] = mn[j] | ((mn[j + 4] >> 4) << 6);
            o[12 + j] = (sc[j + 4] & 0xF) | ((mn[j + 4] & 0xF) << 4);
        }
        uint8_t* qh = o + 16;
        uint8_t* qs = o + (fmt == SLAI_FMT_Q4_K ? 16 : 48);
        if (fmt == SLAI_FMT_Q5_K)
            for (int i = 0; i < 32; i++) qh[i] = 0;
        for (int G = 0; G < 4; G++)
            for (int l = 0; l < 32; l++) {
                int q2[2];
                for (int hf = 0; hf < 2; hf++) {
                    const int j = 2 * G + hf;
                    const float eff = dv * (float)sc[j], off = mv * (float)mn[j];
                    q2[hf] = max(0, min(levels, (int)rintf(sdiv(x[64 * G + 32 * hf + l] + off, eff))));
                }
                qs[32 * G + l] = (uint8_t)((q2[0] & 0xF) | ((q2[1] & 0xF) << 4));
                if (fmt == SLAI_FMT_Q5_K) qh[l] |= (uint8_t)((((q2[0] >> 4) & 1) << (2 * G)) | (((q2[1] >> 4) & 1) << (2 * G + 1)));
            }
        return;
    }
    // Q6_K
    float s[16], smax = 0.f;
    for (int j = 0; j < 16; j++) {
        float amax = 0.f;
        for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(x[16 * j + i]));
        s[j] = amax / 32.0f;
        smax = fmaxf(smax, s[j]);
    }
    const unsigned short db = f2h_bits(smax / 127.0f);
    const float dv = __half2float(__ushort_as_half(db));
    uint8_t* o = out + b * 210;
    int sc[16];
    for (int j = 0; j < 16; j++) {
        sc[j] = max(-128, min(127, (int)rintf(sdiv(s[j], dv))));
        o[192 + j] = (uint8_t)(signed char)sc[j];
    }
    o[208] = db & 0xFF;
    o[209] = db >> 8;
    for (int h = 0; h < 2; h++)
        for (int l = 0; l < 32; l++) {
            int q[4];
            for (int c = 0; c < 4; c++) {
                const int e = 128 * h + 32 * c + l;
                const float eff = dv * (float)sc[e >> 4];
                q[c] = max(-32, min(31, (int)rintf(sdiv(x[e], eff)))) + 32;
            }
            o[64 * h + l] = (uint8_t)((q[0] & 0xF) | ((q[2] & 0xF) << 4));
            o[64 * h + 32 + l] = (uint8_t)((q[1] & 0xF) | ((q[3] & 0xF) << 4));
            o[128 + 32 * h + l] = (uint8_t)((q[0] >> 4) | ((q[1] >> 4) << 2) | ((q[2] >> 4) << 4) | ((q[3] >> 4) << 6));
        }
}

}  // namespace

SLAI_API int slai_synth_blocks(slai_ctx* ctx, int fmt, int64_t nrows, int64_t ncols, uint64_t seed, float std, void* d_blocks) {
    if (!ctx || !d_blocks) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    const int be = fmt_block_elems(fmt);
    SLAI_REQUIRE(ctx, be > 1, SLAI_ERR_UNSUPPORTED_FORMAT, "synth: format %d has no generator", fmt);
    SLAI_REQUIRE(ctx, nrows > 0 && ncols > 0 && ncols % be == 0, SLAI_ERR_SHAPE, "synth: bad shape");
    const long long nblocks = nrows * (ncols / be);
    synth_blocks_kernel<<<(unsigned)((nblocks + 127) / 128), 128, 0, ctx->stream>>>(fmt, (uint8_t*)d_blocks, nblocks, seed, std);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
SLAI_API int slai_synth_normal_f32(slai_ctx* ctx, float* d_out, int64_t n, uint64_t seed, float std) {
    if (!ctx || !d_out || n <= 0) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    synth_normal_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(d_out, n, seed, std);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}

#ifdef SLAI_TRACE
// Trace build only (see common.cuh).  slai_debug_timeline copies the launch records out and restarts the timeline;
// slai_debug_block_trace copies the per-block stamps of the most recent GEMV launch (TRACE_BLOCKS x TRACE_POINTS x u64).
SLAI_API int slai_debug_timeline(slai_ctx* ctx, void* h_out, size_t bytes, unsigned int* count) {
    if (!ctx || !ctx->tl || !h_out || !count) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    const size_t all = (size_t)TL_SLOTS * TL_CAP * 8;
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) return SLAI_ERR_CUDA;
    unsigned long long n = 0;
    if (cudaMemcpy(h_out, ctx->tl, bytes < all ? bytes : all, cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(&n, ctx->tl + TL_SLOTS * TL_CAP, 8, cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemset(ctx->tl + TL_SLOTS * TL_CAP, 0, 8) != cudaSuccess)
        return SLAI_ERR_CUDA;
    *count = (unsigned int)n;
    return SLAI_OK;
}
// The whole ring: 64 launches x TRACE_BLOCKS x TRACE_POINTS stamps; *launches = GEMV launches described so far (the
// launch with index i stamped into slot i % 64).
SLAI_API int slai_debug_trace_ring(slai_ctx* ctx, void* h_out, size_t bytes, unsigned long long* launches) {
    if (!ctx || !ctx->trace_buf || !h_out || !launches) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    const size_t all = (size_t)64 * TRACE_BLOCKS * TRACE_POINTS * 8;
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) return SLAI_ERR_CUDA;
    *launches = ctx->trace_launches;
    return (int)cudaMemcpy(h_out, ctx->trace_buf, bytes < all ? bytes : all, cudaMemcpyDeviceToHost);
}
SLAI_API int slai_debug_block_trace(slai_ctx* ctx, void* h_out, size_t bytes) {
    if (!ctx || !ctx->trace_buf) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    const unsigned long long last = ctx->trace_launches ? (ctx->trace_launches - 1) % 64 : 0;
    const size_t all = (size_t)TRACE_BLOCKS * TRACE_POINTS * 8;
    return (int)cudaMemcpy(h_out, ctx->trace_buf + last * TRACE_BLOCKS * TRACE_POINTS, bytes < all ? bytes : all, cudaMemcpyDeviceToHost);
}
#endif
