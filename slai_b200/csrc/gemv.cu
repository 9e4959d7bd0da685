// Stand-alone fused dequant-GEMV for GGUF Q8_0 / Q4_K / Q5_K / Q6_K weights (GemvQuant::launch,
// crates/slai/src/ops/gemv_quant.rs:206-312) with the decode-path prologues and epilogues fused in:
//   prologue : none | RmsNorm (ops/rms_norm.rs:68-77) | LayerNorm+gamma/beta (ops/layernorm.rs:104-111)
//   epilogue : store | residual add | SiLU gate (ops/silu.rs:50-58) | GELU (ops/unary.rs:81-85) |
//              q/k/v split with RoPE (ops/rope.rs:88-125) and KV-cache append (transformer.rs:329-334)
// The device code (work split, bulk-copy ring, integer tensor-core arithmetic) is in gemv_kernel.cuh; this file
// holds the one-phase kernel, the description of a launch (`fill_params`) and the dispatch over formats.
#include "gemv_kernel.cuh"

using namespace gemvk;

namespace {

template <class F, int NMAT, int PRO, int EPI, bool XIN = false>
__global__ void __launch_bounds__(THREADS, SLAI_GEMV_MINB) gemv_kernel(const __grid_constant__ GemvParams P) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    SLAI_TRACE_POINT(0)
    Ring R;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    ring_setup<F>(R, P, smem_raw, lane, warp);
    SLAI_TRACE_POINT(1)
    // The weights do not depend on the kernel this one may be launched behind (programmatic dependent launch):
    // the ring starts filling while that kernel drains.
    const Split sp = make_split(P);
    ring_fill<F>(R, P, sp, warp);
    SLAI_TRACE_POINT(2)
    // Let the next kernel's blocks be scheduled as this kernel's blocks leave their SMs (it parks in its own
    // griddepcontrol.wait until this grid has completed): the hand-over costs no grid-wide launch latency.
    if (P.pdl == 2) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    prefetch_plan_issue(P.ahead, (int)blockIdx.x, (int)gridDim.x, (int)threadIdx.x, THREADS);
    // Pull data the *next* kernel reads first (its norm weights) into L2 while this one runs.
    if (P.pf_lines > 0 && (int)blockIdx.x == (int)gridDim.x - 1)
        for (int i = threadIdx.x; i < P.pf_lines; i += THREADS) asm volatile("prefetch.global.L2 [%0];" ::"l"(P.pf_ptr + (size_t)i * 128));
    // partial-sum buffer cleared while the predecessor drains
    for (int i = threadIdx.x; i < WAVE * WARPS * NMAT * 16; i += THREADS) reinterpret_cast<float*>(smem_raw + P.dig_region)[i] = 0.f;
    SLAI_TRACE_POINT(3)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    SLAI_TRACE_POINT(4)
    gemv_body<F, NMAT, PRO, EPI, XIN>(P, R, sp, smem_raw);
    if (P.pdl != 2) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#ifdef SLAI_TRACE
    if (blockIdx.x == 0 && threadIdx.x == 0 && P.trace) {
        P.trace[13] = slai_globaltimer();
        slai_tl_append(P.tl, 1000 * (P.K / 256) + 100 * NMAT + 10 * PRO + EPI, P.trace);
    }
#endif
}

// Dense f32 matrix (GpuQuantMatrix::F32): one warp per row.
__global__ void gemv_f32_kernel(float* out, const float* w, const float* v, int M, int K) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= M) return;
    const float* wr = w + (size_t)row * K;
    float acc = 0.f;
    for (int k = lane; k < K; k += 32) acc = fmaf(wr[k], v[k], acc);
    acc = warp_sum(acc);
    if (lane == 0) out[row] = acc;
}

template <class F, int NMAT, int PRO, int EPI, bool XIN = false>
int launch_inst(slai_ctx* ctx, const GemvParams& P, int grid, size_t smem, bool pdl) {
    auto kern = gemv_kernel<F, NMAT, PRO, EPI, XIN>;
    static PerDeviceOnce attr;  // per instantiation
    if (attr.need(ctx->device)) {
        SLAI_CHECK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
        // One shared-memory carve-out for every launch whatever its ring and vector sizes: an SM changes its carve-out
        // only when idle, which would hold back the blocks of the next kernel.
        SLAI_CHECK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        attr.set(ctx->device);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    SLAI_CHECK_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, P));
    return SLAI_OK;
}

template <class F>
int launch_fmt(slai_ctx* ctx, const GemvParams& P, const GemvLaunch& L, int grid, size_t smem) {
    const bool pdl = L.pdl;
#define GO(NMAT, PRO, EPI) return launch_inst<F, NMAT, PRO, EPI>(ctx, P, grid, smem, pdl)
    if (L.xchg_in_idx1 > 0) {  // tensor parallel: the input is an incoming exchange (RmsNorm consumers only)
        if (L.pro == PRO_RMS && L.epi == EPI_QKV) return launch_inst<F, 1, PRO_RMS, EPI_QKV, true>(ctx, P, grid, smem, pdl);
        if (L.pro == PRO_RMS && L.epi == EPI_SILU) return launch_inst<F, 2, PRO_RMS, EPI_SILU, true>(ctx, P, grid, smem, pdl);
        if (L.pro == PRO_RMS && L.epi == EPI_STORE) return launch_inst<F, 1, PRO_RMS, EPI_STORE, true>(ctx, P, grid, smem, pdl);
        return slai_set_error(ctx, SLAI_ERR_INVALID_ARG, "gemv: no kernel consumes an exchange with prologue/epilogue %d/%d", L.pro, L.epi);
    }
    if (L.epi == EPI_XCHG) {
        if (L.pro == PRO_NONE) GO(1, PRO_NONE, EPI_XCHG);
        return slai_set_error(ctx, SLAI_ERR_INVALID_ARG, "gemv: the exchange epilogue takes no prologue");
    }
    switch (L.epi) {
        case EPI_STORE:
            if (L.pro == PRO_NONE) GO(1, PRO_NONE, EPI_STORE);
            if (L.pro == PRO_RMS) GO(1, PRO_RMS, EPI_STORE);
            GO(1, PRO_LN, EPI_STORE);
        case EPI_RESID:
            if (L.pro == PRO_NONE) GO(1, PRO_NONE, EPI_RESID);
            break;
        case EPI_SILU:
            if (L.pro == PRO_RMS) GO(2, PRO_RMS, EPI_SILU);
            if (L.pro == PRO_NONE) GO(2, PRO_NONE, EPI_SILU);
            break;
        case EPI_GELU:
            if (L.pro == PRO_LN) GO(1, PRO_LN, EPI_GELU);
            if (L.pro == PRO_NONE) GO(1, PRO_NONE, EPI_GELU);
            break;
        case EPI_QKV:
            if (L.pro == PRO_RMS) GO(1, PRO_RMS, EPI_QKV);
            if (L.pro == PRO_LN) GO(1, PRO_LN, EPI_QKV);
            if (L.pro == PRO_NONE) GO(1, PRO_NONE, EPI_QKV);
            break;
    }
#undef GO
    return slai_set_error(ctx, SLAI_ERR_INVALID_ARG, "gemv: unsupported prologue/epilogue combination %d/%d", L.pro, L.epi);
}

}  // namespace

// Bytes of shared memory the staged activation vector of a K-element phase needs (zero page, digit planes, digit
// sums: 16 bytes per sub-block in both representations of gemv_formats.cuh).
size_t gemv_dig_region(int fmt, int K) {
    const int Kp = (K + 255) & ~255;
    const int sv_gran = (fmt == SLAI_FMT_Q4_K || fmt == SLAI_FMT_Q5_K) ? 32 : fmt == SLAI_FMT_Q6_K ? 16 : 0;
    const size_t sv_bytes = sv_gran ? (size_t)(Kp / sv_gran) * 16 : 0;
    return ((size_t)gemvfmt::ZERO_BYTES + ((size_t)4 * (Kp + 32) + sv_bytes) + 127) & ~(size_t)127;
}

// Validate a launch description and turn it into kernel parameters.  `dig_region` = 0: size it for this K.
int gemv_fill_params(slai_ctx* ctx, const GemvLaunch& L, size_t dig_region, int nstage, GemvParams& P, size_t* smem_out,
                     int* grid_out) {
    const int K = L.K;
    const int be = fmt_block_elems(L.fmt);
    SLAI_REQUIRE(ctx, be > 0 && L.fmt != SLAI_FMT_F32, SLAI_ERR_UNSUPPORTED_FORMAT, "gemv: format %d has no kernel", L.fmt);
    SLAI_REQUIRE(ctx, K > 0 && K % be == 0, SLAI_ERR_SHAPE, "gemv: K=%d is not a multiple of the block size %d", K, be);
    SLAI_REQUIRE(ctx, ((uintptr_t)L.v & 15) == 0, SLAI_ERR_INVALID_ARG, "gemv: input vector must be 16-byte aligned");
    P = GemvParams{};
    P.nseg = L.nseg;
    int tiles = 0;
    for (int s = 0; s < L.nseg; s++) {
        P.seg[s] = L.seg[s];
        P.seg[s].tile0 = tiles;
        tiles += (L.seg[s].rows + 15) / 16;
        SLAI_REQUIRE(ctx, ((uintptr_t)L.seg[s].w & 15) == 0, SLAI_ERR_INVALID_ARG, "gemv: matrix data must be 16-byte aligned");
    }
    const bool dual = (L.epi == EPI_SILU);
    P.nmat = dual ? 2 : 1;
    if (dual) {
        SLAI_REQUIRE(ctx, L.nseg == 2 && L.seg[0].rows == L.seg[1].rows, SLAI_ERR_SHAPE, "gemv: gate/up shapes differ");
        P.n_items = (L.seg[0].rows + 15) / 16;
    } else {
        P.n_items = tiles;
    }
    if (L.epi == EPI_QKV) {
        SLAI_REQUIRE(ctx, L.head_size > 0 && L.head_size % 2 == 0 && L.d_pos, SLAI_ERR_INVALID_ARG, "gemv: bad q/k/v arguments");
        SLAI_REQUIRE(ctx, !L.rope || L.rope_theta, SLAI_ERR_INVALID_ARG, "gemv: RoPE table missing");
    }
    P.K = K;
    P.nsteps = (int)layout::num_steps(L.fmt, K);
    P.step_bytes = layout::step_bytes(L.fmt);
    P.stage_stride = (P.step_bytes + 8 + 127) & ~127;  // block + its mbarrier (RingGeom)
    P.v = L.v; P.out = L.out; P.norm_w = L.norm_w; P.norm_b = L.norm_b; P.eps = L.eps;
    P.resid = L.resid; P.rope = L.rope; P.rope_theta = L.rope_theta; P.rope_cs = L.rope_cs; P.head_size = L.head_size;
    P.d_pos = L.d_pos; P.pos1 = 0; P.kcache = L.kcache; P.vcache = L.vcache; P.k_out = L.k_out; P.kv_f16 = (L.kv_dtype == SLAI_KV_F16);
    P.kv_pos_stride = L.kv_pos_stride; P.kv_head_stride = L.kv_head_stride;
    P.err_flag = ctx->d_counters + CNT_ERR_FLAG;
    P.wait_limit = ctx->wait_limit;
    static int pdl_early = -1;
    if (pdl_early < 0) {
        const char* e = getenv("SLAI_PDL_EARLY");
        pdl_early = (e && e[0] == '0') ? 0 : 1;
    }
    P.pdl = L.pdl ? (pdl_early ? 2 : 1) : 0;
    P.pf_ptr = reinterpret_cast<const char*>(L.prefetch);
    P.pf_lines = L.prefetch ? (int)((L.prefetch_bytes + 127) / 128) : 0;
    P.ahead = L.ahead;
    P.xr = 0;
    P.xi_slots = nullptr;
    P.xl_sum = nullptr;
    if (L.xchg) {
        const PeerExchange& X = *L.xchg;
        SLAI_REQUIRE(ctx, X.ranks >= 2 && X.ranks <= XCHG_MAX_RANKS, SLAI_ERR_INVALID_ARG, "gemv: exchange group of %d ranks", X.ranks);
        P.xr = X.ranks;
        P.xrank = X.rank;
        P.x_tokseq = X.d_tokseq;
        P.x_per_token = (unsigned int)L.xchg_per_token;
        P.xo_idx1 = (unsigned int)L.xchg_out_idx1;
        P.xi_idx1 = (unsigned int)L.xchg_in_idx1;
        P.xsum_out = L.xsum_out;
        if (L.epi == EPI_XCHG) {
            SLAI_REQUIRE(ctx, L.xchg_out_idx1 > 0 && L.nseg == 1 && L.seg[0].rows <= XCHG_MAX_DIM, SLAI_ERR_SHAPE, "gemv: bad outgoing exchange");
            const int par = (L.xchg_out_idx1 - 1) & 1;
            for (int r = 0; r < X.ranks; r++) P.xo_slot[r] = X.slot_at[r] + ((size_t)par * X.ranks + X.rank) * XCHG_MAX_DIM;
        }
        if (L.xchg_in_idx1 > 0) {
            SLAI_REQUIRE(ctx, K <= XCHG_MAX_DIM && (K >> 2) <= STAGE_REGS * THREADS && L.xsum_out, SLAI_ERR_SHAPE,
                         "gemv: incoming exchange of %d floats does not fit the staging registers", K);
            const int par = (L.xchg_in_idx1 - 1) & 1;
            P.xi_slots = X.slot_at[X.rank] + (size_t)par * X.ranks * XCHG_MAX_DIM;
            // Group size from which the blocks share one sum (SLAI_TP_TWO_LEVEL=<ranks>).  Off by default: measured at
            // eight ranks the two-level sum (6.18 ms per 70B token) does not beat every block summing all ranks' partials
            // itself (5.99 ms); the extra local round trip costs what the smaller L2 volume saves.
            static int two_level_from = -1;
            if (two_level_from < 0) {
                const char* e = getenv("SLAI_TP_TWO_LEVEL");
                two_level_from = e ? atoi(e) : 1 << 30;
            }
            P.xl_sum = X.ranks >= two_level_from ? X.local_sum + (size_t)par * XCHG_MAX_DIM : nullptr;
        }
    }
#ifdef SLAI_TRACE
    // every launch stamps into its own slot of a 64-deep ring: consecutive kernels overlap under dependent launch
    P.trace = ctx->trace_buf + (size_t)(ctx->trace_launches++ % 64) * TRACE_BLOCKS * TRACE_POINTS;
    P.tl = ctx->tl;
#endif
    const size_t need = gemv_dig_region(L.fmt, K);
    if (dig_region == 0) dig_region = need;
    SLAI_REQUIRE(ctx, dig_region >= need, SLAI_ERR_INVALID_ARG, "gemv: staging region too small");
    P.dig_region = (int)dig_region;
    const size_t fixed = dig_region + (size_t)RED_FLOATS * 4 + 64 * 4 + 128;
    const size_t per_stage = (size_t)WARPS * P.stage_stride;
    if (nstage <= 0) {
        SLAI_REQUIRE(ctx, fixed + 2 * per_stage <= SMEM_LIMIT, SLAI_ERR_SHAPE, "gemv: K=%d does not fit in shared memory", K);
        const int fit = (int)((SMEM_LIMIT - fixed) / per_stage);
        // Two stages in flight per warp for the K-quants (three otherwise) measured fastest: a deeper first fill asks for
        // most of the matrix at once and delays the activation loads of the staging pass behind it.
        const bool kquant = L.fmt == SLAI_FMT_Q4_K || L.fmt == SLAI_FMT_Q5_K || L.fmt == SLAI_FMT_Q6_K;
        nstage = kquant ? 2 : 3;
        static int stage_env = -1;
        if (stage_env < 0) {
            const char* e = getenv("SLAI_GEMV_STAGES");
            stage_env = e ? atoi(e) : 0;
        }
        if (stage_env >= 2) nstage = stage_env;
        if (nstage > fit) nstage = fit;
        if (nstage > MAX_STAGES) nstage = MAX_STAGES;
    }
    P.nstage = nstage;
    if (smem_out) *smem_out = fixed + (size_t)nstage * per_stage;
    const int grid = P.n_items < ctx->sm_count ? P.n_items : ctx->sm_count;
    P.items_base = P.n_items / grid;
    P.items_rem = P.n_items % grid;
    if (grid_out) *grid_out = grid;
    return SLAI_OK;
}

static int gemv_launch_inner(slai_ctx* ctx, const GemvLaunch& L);
int gemv_launch(slai_ctx* ctx, const GemvLaunch& L) {
    if (!ctx->stats_on) return gemv_launch_inner(ctx, L);
    // statistics: what ran since the last mark is "other"; this kernel's class follows from its epilogue
    int rc = slai_stats_mark(ctx, STATS_OTHER);
    if (rc) return rc;
    if ((rc = gemv_launch_inner(ctx, L))) return rc;
    const int cls = L.stats_cls >= 0 ? L.stats_cls : L.epi == EPI_QKV ? STATS_QKV : L.epi == EPI_SILU ? STATS_GATE_UP
                    : (L.epi == EPI_RESID || L.epi == EPI_XCHG) ? STATS_WO : STATS_OTHER;
    return slai_stats_mark(ctx, cls);
}
static int gemv_launch_inner(slai_ctx* ctx, const GemvLaunch& L) {
    const int K = L.K;
    if (L.fmt == SLAI_FMT_F32) {
        SLAI_REQUIRE(ctx, L.nseg == 1 && L.pro == PRO_NONE && L.epi == EPI_STORE && !L.seg[0].bias, SLAI_ERR_INVALID_ARG,
                     "gemv: dense f32 matrices support only the plain product");
        const int M = L.seg[0].rows;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((M + 7) / 8);
        cfg.blockDim = dim3(256);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = L.pdl ? 1 : 0;
        SLAI_CHECK_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemv_f32_kernel, L.out, (const float*)L.seg[0].w, L.v, M, K));
        return SLAI_OK;
    }
    GemvParams P;
    size_t smem = 0;
    int grid = 0;
    int rc = gemv_fill_params(ctx, L, 0, 0, P, &smem, &grid);
    if (rc) return rc;
    switch (L.fmt) {
        case SLAI_FMT_Q4_K: return launch_fmt<Q4K>(ctx, P, L, grid, smem);
        case SLAI_FMT_Q5_K: return launch_fmt<Q5K>(ctx, P, L, grid, smem);
        case SLAI_FMT_Q6_K: return launch_fmt<Q6K>(ctx, P, L, grid, smem);
        case SLAI_FMT_Q8_0: return launch_fmt<Q80>(ctx, P, L, grid, smem);
    }
    return slai_set_error(ctx, SLAI_ERR_UNSUPPORTED_FORMAT, "gemv: format %d has no kernel", L.fmt);
}
