// Per-token decode of the Llama-2 family (Llama2::launch, crates/slai/src/models/llama2/transformer.rs:316-381;
// caller ChatLlama2::forward_logits, crates/slai-chat/src/chat_llama2.rs:163-240) and of GPT-2
// (gpt2::cpu::Transformer::forward, crates/slai/src/models/gpt2/cpu.rs:225-383).
//
// The reference records ~16 dispatches per layer and synchronises + reads back all logits per token.
// Here a layer is five kernels (norm+QKV+RoPE+KV-append, attention, O+residual, norm+gate/up+SiLU,
// down+residual), chained with programmatic dependent launch and captured once into a CUDA graph that is
// replayed per token; token id and position live in device scalars, and greedy decoding / prompt
// processing advance them on the device so the host only launches graphs.
#include <algorithm>

#include "common.cuh"

namespace {

struct Scalars {  // device ints: [0] token, [1] pos, [2] step, [3] next
    int* d = nullptr;
};

enum GraphKind { G_DECODE = 0, G_GENERATE = 1, G_FORCED = 2, G_SAMPLED = 3, G_COUNT = 4 };

struct GraphSet {
    cudaGraphExec_t exec[G_COUNT] = {};
    bool warmed[G_COUNT] = {};  // first token of a kind runs eagerly (sets kernel attributes)
    bool use_graph = true;
};

int copy_f32(slai_ctx* ctx, float** dst, const float* src, int64_t n, bool from_device) {
    if (*dst) {
        cudaStreamSynchronize(ctx->stream);
        cudaFree(*dst);
        *dst = nullptr;
    }
    SLAI_CHECK_CUDA(ctx, cudaMalloc(dst, (size_t)n * 4 + 16));
    SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(*dst, src, (size_t)n * 4, from_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice,
                                         ctx->stream));
    SLAI_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return SLAI_OK;
}

void destroy_graphs(GraphSet& g) {
    for (int i = 0; i < G_COUNT; i++)
        if (g.exec[i]) {
            cudaGraphExecDestroy(g.exec[i]);
            g.exec[i] = nullptr;
        }
    for (int i = 0; i < G_COUNT; i++) g.warmed[i] = false;
}

// Bytes of later weights one kernel asks for ahead of time (PrefetchPlan).  Off unless SLAI_AHEAD_MB is set: the main
// loop consumes no faster from L2 than from HBM, so requests issued ahead only lengthen the hand-over (measured).
size_t ahead_cap_bytes() {
    static long long cap = -1;
    if (cap < 0) {
        const char* e = getenv("SLAI_AHEAD_MB");
        cap = (e ? atoll(e) : 0) << 20;
    }
    return (size_t)cap;
}
// Plan for bytes [from, from + cap) of the concatenation of up to three quantised matrices, taken in equal shares
// from each (they are streamed side by side: q/k/v tiles in turn, gate and up tile by tile).
PrefetchPlan plan_ahead(const slai_qmatrix* const* ms, int n, size_t from_each, size_t cap) {
    PrefetchPlan p;
    if (cap == 0 || n <= 0) return p;
    size_t total = 0;
    for (int i = 0; i < n; i++) total += (ms[i] && ms[i]->fmt != SLAI_FMT_F32 && ms[i]->bytes > from_each) ? ms[i]->bytes - from_each : 0;
    if (total == 0) return p;
    for (int i = 0; i < n && i < 3; i++) {
        if (!ms[i] || ms[i]->fmt == SLAI_FMT_F32 || ms[i]->bytes <= from_each) continue;
        const size_t avail = ms[i]->bytes - from_each;
        size_t take = total <= cap ? avail : (size_t)((double)avail * (double)cap / (double)total);
        take &= ~(size_t)15;
        p.ptr[i] = reinterpret_cast<const char*>(ms[i]->data) + (from_each & ~(size_t)15);
        p.bytes[i] = take;
    }
    return p;
}
PrefetchPlan plan_ahead1(const slai_qmatrix* m, size_t from, size_t cap) { return plan_ahead(&m, 1, from, cap); }

GemvSeg seg_of(const slai_qmatrix* m, int row0, int rows, const float* bias, int out_off, int role) {
    GemvSeg s;  // row0 is a multiple of 16 (checked where fused matrices are attached)
    s.w = m->fmt == SLAI_FMT_F32 ? m->data + (size_t)row0 * m->tile_bytes : m->data + (size_t)(row0 / 16) * m->tile_bytes;
    s.tile_bytes = m->tile_bytes;
    s.rows = rows;
    s.bias = bias;
    s.out_off = out_off;
    s.role = role;
    return s;
}

}  // namespace

// =================================================================================================
// Llama
// =================================================================================================
struct LlamaLayer {
    const slai_qmatrix *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr, *wgate = nullptr, *wup = nullptr,
                       *wdown = nullptr;
    float *attn_norm = nullptr, *ffn_norm = nullptr, *bq = nullptr, *bk = nullptr, *bv = nullptr;
};

struct slai_llama {
    slai_ctx* ctx = nullptr;
    slai_llama_config cfg;
    int kv_dim = 0, head_size = 0, kv_mul = 0;  // kv_dim: this rank's share
    // tensor-parallel shares of this rank (equal to the global sizes when tp_size == 1): query rows, query heads,
    // FFN rows; x (dim floats) is replicated, xpart receives a row-parallel GEMV's partial before the exchange
    int q_dim = 0, n_q_local = 0, hidden = 0, tp = 1;
    float* xpart = nullptr;
    float* rope_cs = nullptr;  // (cos, sin) of the current token's RoPE angles, written by the embedding kernel
    void *d_samp = nullptr, *d_samp_scratch = nullptr;  // sampler parameters and sort scratch (slai_llama_generate_sampled)
    std::vector<LlamaLayer> layers;
    const slai_qmatrix* output = nullptr;
    const slai_qmatrix* embd_q = nullptr;
    slai_qmatrix embd_as_matrix;  // non-owning F32 view of the f32 embedding table (tied output)
    float* token_embd = nullptr;  // [vocab][dim] f32
    float* out_norm = nullptr;
    float *x = nullptr, *xb = nullptr, *q = nullptr, *hb = nullptr, *hb2 = nullptr, *logits = nullptr;
    float *ktmp = nullptr, *vtmp = nullptr;  // k / v of the current token as f32 where the fused q/k/v epilogue cannot write the cache itself
    float* logits_part = nullptr;  // tensor parallel with a row-sharded output matrix: this rank's vocab / tp logits
    bool out_sharded = false;
    void *kcache = nullptr, *vcache = nullptr;
    size_t kv_layer_elems = 0;
    Scalars sc;
    int32_t* d_history = nullptr;  // generated / forced token ids
    int history_cap = 0;
    void* attn_scratch = nullptr;
    size_t attn_scratch_bytes = 0;
    const float* rope_theta = nullptr;
    GraphSet graphs;
    int launches = 0;
    // prompt processing as GEMMs (prefill.cu): buffers for `pf_cap` tokens, grown on demand
    int pf_cap = 0, pf_attn_batch = 0;
    float *pf_x = nullptr, *pf_qkv = nullptr, *pf_q = nullptr, *pf_xb = nullptr, *pf_g = nullptr, *pf_u = nullptr;
    float* pf_part = nullptr;  // sharded models: this rank's partial of a row-parallel product, [tokens][dim]
    __half *pf_hi = nullptr, *pf_lo = nullptr;
    int* pf_tokens = nullptr;
    void* pf_attn_scratch = nullptr;
    size_t pf_attn_scratch_bytes = 0;
    unsigned int* pf_tickets = nullptr;
    // several sequences decoded together (slai_llama_decode_batch): one KV cache per sequence, activations of all of them
    int bt_n = 0;
    void *bt_k = nullptr, *bt_v = nullptr;  // [sequence][layer][kv head][position][head_size]
    size_t bt_cache_bytes = 0;              // per sequence
    float *bt_x = nullptr, *bt_xn = nullptr, *bt_q = nullptr, *bt_qkv = nullptr, *bt_xb = nullptr, *bt_t = nullptr, *bt_g = nullptr,
          *bt_u = nullptr, *bt_logits = nullptr;
    int* bt_i = nullptr;  // device ints: [0, 8) tokens, [8, 16) positions, [16, 24) greedy choices
    void* bt_attn = nullptr;  // attention partials of all sequences
    unsigned int* bt_tickets = nullptr;
    // the step of n sequences as a replayed graph (index n), captured for contexts up to bt_cap[n] positions
    cudaGraphExec_t bt_exec[9] = {};
    int bt_cap[9] = {};
    bool bt_warm[9] = {};
};

static void llama_drop_batch_graphs(slai_llama* m) {
    for (int i = 0; i < 9; i++) {
        if (m->bt_exec[i]) cudaGraphExecDestroy(m->bt_exec[i]);
        m->bt_exec[i] = nullptr;
        m->bt_cap[i] = 0;
        m->bt_warm[i] = false;
    }
}

static void llama_drop_batch(slai_llama* m) {
    if (m->bt_n) cudaStreamSynchronize(m->ctx->stream);
    llama_drop_batch_graphs(m);
    cudaFree(m->bt_k); cudaFree(m->bt_v); cudaFree(m->bt_x); cudaFree(m->bt_xn); cudaFree(m->bt_q); cudaFree(m->bt_qkv);
    cudaFree(m->bt_xb); cudaFree(m->bt_t); cudaFree(m->bt_g); cudaFree(m->bt_u); cudaFree(m->bt_logits); cudaFree(m->bt_i);
    cudaFree(m->bt_attn); cudaFree(m->bt_tickets);
    m->bt_k = m->bt_v = m->bt_attn = nullptr;
    m->bt_x = m->bt_xn = m->bt_q = m->bt_qkv = m->bt_xb = m->bt_t = m->bt_g = m->bt_u = m->bt_logits = nullptr;
    m->bt_i = nullptr;
    m->bt_tickets = nullptr;
    m->bt_n = 0;
}

static void llama_drop_prefill(slai_llama* m) {
    if (m->pf_cap) cudaStreamSynchronize(m->ctx->stream);
    cudaFree(m->pf_x); cudaFree(m->pf_qkv); cudaFree(m->pf_q); cudaFree(m->pf_xb); cudaFree(m->pf_g); cudaFree(m->pf_u);
    cudaFree(m->pf_hi); cudaFree(m->pf_lo); cudaFree(m->pf_tokens); cudaFree(m->pf_attn_scratch); cudaFree(m->pf_tickets);
    cudaFree(m->pf_part);
    m->pf_x = m->pf_qkv = m->pf_q = m->pf_xb = m->pf_g = m->pf_u = m->pf_part = nullptr;
    m->pf_hi = m->pf_lo = nullptr;
    m->pf_tokens = nullptr;
    m->pf_attn_scratch = nullptr;
    m->pf_attn_scratch_bytes = 0;
    m->pf_tickets = nullptr;
    m->pf_cap = 0;
}

static int llama_record(slai_llama* m, int kind) {
    slai_ctx* ctx = m->ctx;
    const slai_llama_config& c = m->cfg;
    const bool pdl = ctx->use_pdl;
    int n = 0;
    int* d_token = m->sc.d;
    int* d_pos = m->sc.d + 1;
    int rc;
    SLAI_REQUIRE(ctx, m->out_norm && (m->token_embd || m->embd_q), SLAI_ERR_INVALID_ARG, "llama: embedding / output norm not set");
    const bool table = c.rope_variant == 0 && m->head_size / 2 <= 256;
    if (m->embd_q) rc = launch_embed_q8(ctx, m->x, m->embd_q, d_token, nullptr, d_pos, false, m->rope_theta, table ? m->rope_cs : nullptr, m->head_size / 2);
    else rc = launch_embed_f32(ctx, m->x, m->token_embd, c.dim, d_token, nullptr, d_pos, false, m->rope_theta, table ? m->rope_cs : nullptr, m->head_size / 2);
    if (rc) return rc;
    n++;
    const size_t esz = c.kv_dtype == SLAI_KV_F16 ? 2 : 4;
    // A row-parallel GEMV (each rank holds a K range of every row): x += W v.  Sharded: the partial goes to xpart
    // (rank 0 adds the residual), then one sum over the ranks writes x on every rank.
    // With the ranks' exchange regions mapped into each other (slai_tp_peer_attach) there is no collective at
    // all: the row-parallel GEMV stores its partial rows into every rank's region (EPI_XCHG) and the next GEMV
    // sums them while staging its input (xchg_in), leaving the new x behind for the residual of the one after.
    bool use_x = m->tp > 1 && ctx->xchg_ready && c.dim <= XCHG_MAX_DIM && c.dim <= 12288;
    {
        const char* e = getenv("SLAI_TP_NCCL");
        if (e && e[0] == '1') use_x = false;
        const slai_qmatrix* wo_ = m->output ? m->output : (m->embd_q ? m->embd_q : &m->embd_as_matrix);
        if (wo_->fmt == SLAI_FMT_F32) use_x = false;
        for (auto& w : m->layers)
            if (!w.wq || !w.wk || !w.wv || !w.wgate || !w.wup || w.wq->fmt != w.wk->fmt || w.wk->fmt != w.wv->fmt || w.wgate->fmt != w.wup->fmt)
                use_x = false;
    }
    int xi = 0;  // exchanges issued so far in this token
    if (use_x) {
        if ((rc = tp_tick(ctx))) return rc;
        n++;
    }
    auto consume_exchange = [&](GemvLaunch& L) {  // the input of L is the sum of the last exchange
        if (use_x && xi > 0) {
            L.xchg = &ctx->xchg;
            L.xchg_in_idx1 = xi;
            L.xchg_per_token = 2 * c.n_layers;
            L.xsum_out = m->x;
        }
    };
    auto row_parallel = [&](GemvLaunch& L) -> int {
        int r;
        if (m->tp == 1) {
            n++;
            return gemv_launch(ctx, L);
        }
        if (use_x) {
            L.xchg = &ctx->xchg;
            L.epi = EPI_XCHG;
            L.xchg_out_idx1 = ++xi;
            L.xchg_per_token = 2 * c.n_layers;
            n++;
            return gemv_launch(ctx, L);
        }
        L.out = m->xpart;
        if (ctx->tp_rank != 0) {
            L.resid = nullptr;
            L.epi = EPI_STORE;
        }
        if ((r = gemv_launch(ctx, L))) return r;
        if ((r = tp_all_reduce_sum(ctx, m->xpart, m->x, c.dim))) return r;
        n += 2;
        return SLAI_OK;
    };
    for (int l = 0; l < c.n_layers; l++) {
        const LlamaLayer& w = m->layers[l];
        SLAI_REQUIRE(ctx, w.wq && w.wk && w.wv && w.wo && w.wgate && w.wup && w.wdown && w.attn_norm && w.ffn_norm,
                     SLAI_ERR_INVALID_ARG, "llama: layer %d has unset weights", l);
        void* kc = (char*)m->kcache + (size_t)l * m->kv_layer_elems * esz;
        void* vc = (char*)m->vcache + (size_t)l * m->kv_layer_elems * esz;
        // Weights are requested one kernel ahead (PrefetchPlan): QKV asks for Wo, attention for the first `cap` bytes of
        // gate / up, O for their rest, gate/up for Wdown, Wdown for the next layer's q / k / v.
        const size_t cap = ahead_cap_bytes();
        const slai_qmatrix* gu[2] = {w.wgate, w.wup};
        const size_t gu_total = (w.wgate ? w.wgate->bytes : 0) + (w.wup ? w.wup->bytes : 0);
        const size_t gu_first = gu_total <= cap ? (size_t)-1 >> 1 : (size_t)((double)(w.wgate ? w.wgate->bytes : 0) * (double)cap / (double)gu_total) & ~(size_t)15;
        // 1. xb = rmsnorm(x); q = Wq xb; k,v -> cache[pos]; RoPE(q,k)          transformer.rs:327-347
        const bool fuse_rope = c.rope_variant == 0;
        const bool dense = w.wq->fmt == SLAI_FMT_F32 || w.wk->fmt == SLAI_FMT_F32 || w.wv->fmt == SLAI_FMT_F32 || w.wo->fmt == SLAI_FMT_F32 ||
                           w.wgate->fmt == SLAI_FMT_F32 || w.wup->fmt == SLAI_FMT_F32 || w.wdown->fmt == SLAI_FMT_F32;
        if (dense) {
            // Dense f32 matrices (the legacy formats that are dequantised at upload, or f32 tensors of a file) have no fused
            // prologues / epilogues: the layer is the reference's own operator sequence, one kernel each
            // (transformer.rs:327-365), on the device-side position.
            SLAI_REQUIRE(ctx, m->tp == 1, SLAI_ERR_INVALID_ARG, "llama: dense f32 layer matrices are not sharded");
            auto plain = [&](const slai_qmatrix* wm, int rows, const float* v, float* out, const float* bias) -> int {
                GemvLaunch L;
                L.fmt = wm->fmt; L.K = (int)wm->ncols; L.nseg = 1; L.seg[0] = seg_of(wm, 0, rows, wm->fmt == SLAI_FMT_F32 ? nullptr : bias, 0, 0);
                L.v = v; L.out = out; L.epi = EPI_STORE; L.pdl = false;
                int r = gemv_launch(ctx, L);
                n++;
                if (!r && bias && wm->fmt == SLAI_FMT_F32) {
                    r = slai_add_assign(ctx, out, bias, rows);
                    n++;
                }
                return r;
            };
            if ((rc = slai_rms_norm(ctx, m->xb, m->x, w.attn_norm, c.dim, c.rms_norm_eps))) return rc;
            if ((rc = plain(w.wq, m->q_dim, m->xb, m->q, w.bq))) return rc;
            if ((rc = plain(w.wk, m->kv_dim, m->xb, m->ktmp, w.bk))) return rc;
            if ((rc = plain(w.wv, m->kv_dim, m->xb, m->vtmp, w.bv))) return rc;
            if ((rc = rope_kv_store_launch(ctx, m->q, m->ktmp, m->vtmp, m->q_dim, m->kv_dim, m->head_size, d_pos, m->rope_theta, c.rope_variant != 0,
                                           kc, vc, c.kv_dtype == SLAI_KV_F16, (long long)c.seq_len * m->head_size, false)))
                return rc;
            n += 2;
            {
                AttnLaunch A;
                A.q = m->q; A.kcache = kc; A.vcache = vc; A.kv_dtype = c.kv_dtype;
                A.pos_stride = m->head_size; A.head_stride = (int64_t)c.seq_len * m->head_size;
                A.n_heads = m->n_q_local; A.kv_mul = m->kv_mul; A.head_size = m->head_size;
                A.d_pos = d_pos; A.max_pos = c.seq_len - 1; A.out = m->xb; A.pdl = false;
                A.scratch = m->attn_scratch; A.scratch_bytes = m->attn_scratch_bytes;
                if ((rc = attention_launch(ctx, A))) return rc;
                n++;
            }
            if ((rc = plain(w.wo, c.dim, m->xb, m->xpart, nullptr))) return rc;
            if ((rc = slai_add_assign(ctx, m->x, m->xpart, c.dim))) return rc;
            if ((rc = slai_rms_norm(ctx, m->xb, m->x, w.ffn_norm, c.dim, c.rms_norm_eps))) return rc;
            if ((rc = plain(w.wgate, m->hidden, m->xb, m->hb, nullptr))) return rc;
            if ((rc = plain(w.wup, m->hidden, m->xb, m->hb2, nullptr))) return rc;
            if ((rc = slai_silu_gate(ctx, m->hb, m->hb2, m->hidden))) return rc;
            if ((rc = plain(w.wdown, c.dim, m->hb, m->xpart, nullptr))) return rc;
            if ((rc = slai_add_assign(ctx, m->x, m->xpart, c.dim))) return rc;
            n += 4;
            continue;
        }
        auto qkv_launch = [&](int nseg, const GemvSeg* segs, int fmt) {
            GemvLaunch L;
            L.fmt = fmt; L.K = c.dim; L.nseg = nseg;
            for (int i = 0; i < nseg; i++) L.seg[i] = segs[i];
            L.v = m->x; L.out = m->q; L.pro = PRO_RMS; L.norm_w = w.attn_norm; L.eps = c.rms_norm_eps;
            L.epi = EPI_QKV; L.rope = fuse_rope ? 1 : 0; L.rope_theta = m->rope_theta; L.head_size = m->head_size;
            L.rope_cs = table ? m->rope_cs : nullptr;
            L.d_pos = d_pos; L.kcache = kc; L.vcache = vc; L.kv_dtype = c.kv_dtype;
            L.kv_pos_stride = m->head_size; L.kv_head_stride = (int64_t)c.seq_len * m->head_size;
            L.k_out = fuse_rope ? nullptr : m->ktmp;  // NeoX pairs rows half a head apart: rotated by the kernel that follows
            L.pdl = pdl;
            L.ahead = plan_ahead1(w.wo, 0, cap);  // the attention kernel in between streams the KV cache, not weights
            consume_exchange(L);
            n++;
            return gemv_launch(ctx, L);
        };
        GemvSeg sq = seg_of(w.wq, 0, m->q_dim, w.bq, 0, 0), sk = seg_of(w.wk, 0, m->kv_dim, w.bk, 0, 1),
                sv = seg_of(w.wv, 0, m->kv_dim, w.bv, 0, 2);
        if (w.wq->fmt == w.wk->fmt && w.wk->fmt == w.wv->fmt) {
            GemvSeg s3[3] = {sq, sk, sv};
            if ((rc = qkv_launch(3, s3, w.wq->fmt))) return rc;
        } else {
            if ((rc = qkv_launch(1, &sq, w.wq->fmt))) return rc;
            if ((rc = qkv_launch(1, &sk, w.wk->fmt))) return rc;
            if ((rc = qkv_launch(1, &sv, w.wv->fmt))) return rc;
        }
        if (!fuse_rope) {  // NeoX (rope.slang:58-86; variant chosen per model, transformer.rs:346-347): q in place, k into the cache
            if ((rc = rope_kv_store_launch(ctx, m->q, m->ktmp, nullptr, m->q_dim, m->kv_dim, m->head_size, d_pos, m->rope_theta, 1, kc, vc,
                                           c.kv_dtype == SLAI_KV_F16, (long long)c.seq_len * m->head_size, pdl)))
                return rc;
            n++;
        }
        // 2. xb = attention(q, cache)                                           transformer.rs:350,383-400
        {
            AttnLaunch A;
            A.q = m->q; A.kcache = kc; A.vcache = vc; A.kv_dtype = c.kv_dtype;
            A.pos_stride = m->head_size; A.head_stride = (int64_t)c.seq_len * m->head_size;
            A.n_heads = m->n_q_local; A.kv_mul = m->kv_mul; A.head_size = m->head_size;
            A.d_pos = d_pos; A.max_pos = c.seq_len - 1; A.out = m->xb; A.pdl = pdl; A.pos_stable = true;
            A.scratch = m->attn_scratch; A.scratch_bytes = m->attn_scratch_bytes;
            A.ahead = plan_ahead(gu, 2, 0, cap);
            if ((rc = attention_launch(ctx, A))) return rc;
            n++;
        }
        // 3. x += Wo xb                                                         transformer.rs:352-355
        {
            GemvLaunch L;
            L.fmt = w.wo->fmt; L.K = m->q_dim; L.nseg = 1; L.seg[0] = seg_of(w.wo, 0, c.dim, nullptr, 0, 0);
            L.v = m->xb; L.out = m->x; L.resid = m->x; L.epi = EPI_RESID; L.pdl = pdl;
            L.prefetch = w.ffn_norm; L.prefetch_bytes = (size_t)c.dim * 4;
            L.ahead = plan_ahead(gu, 2, gu_first, cap);  // what the attention kernel's plan left of gate / up
            if ((rc = row_parallel(L))) return rc;
        }
        // 4. xb = rmsnorm(x); hb = silu(Wgate xb) * (Wup xb)                    transformer.rs:356-361
        if (w.wgate->fmt == w.wup->fmt) {
            GemvLaunch L;
            L.fmt = w.wgate->fmt; L.K = c.dim; L.nseg = 2;
            L.seg[0] = seg_of(w.wgate, 0, m->hidden, nullptr, 0, 0);
            L.seg[1] = seg_of(w.wup, 0, m->hidden, nullptr, 0, 0);
            L.v = m->x; L.out = m->hb; L.pro = PRO_RMS; L.norm_w = w.ffn_norm; L.eps = c.rms_norm_eps; L.epi = EPI_SILU;
            L.pdl = pdl;
            L.ahead = plan_ahead1(w.wdown, 0, cap);
            consume_exchange(L);
            if ((rc = gemv_launch(ctx, L))) return rc;
            n++;
        } else {
            for (int i = 0; i < 2; i++) {
                const slai_qmatrix* wm = i == 0 ? w.wgate : w.wup;
                GemvLaunch L;
                L.fmt = wm->fmt; L.K = c.dim; L.nseg = 1; L.seg[0] = seg_of(wm, 0, m->hidden, nullptr, 0, 0);
                L.v = m->x; L.out = i == 0 ? m->hb : m->hb2; L.pro = PRO_RMS; L.norm_w = w.ffn_norm; L.eps = c.rms_norm_eps;
                L.epi = EPI_STORE; L.pdl = pdl;
                if ((rc = gemv_launch(ctx, L))) return rc;
                n++;
            }
            if ((rc = slai_silu_gate(ctx, m->hb, m->hb2, m->hidden))) return rc;
            n++;
        }
        // 5. x += Wdown hb                                                      transformer.rs:362-365
        {
            GemvLaunch L;
            L.fmt = w.wdown->fmt; L.K = m->hidden; L.nseg = 1; L.seg[0] = seg_of(w.wdown, 0, c.dim, nullptr, 0, 0);
            L.v = m->hb; L.out = m->x; L.resid = m->x; L.epi = EPI_RESID; L.pdl = pdl; L.stats_cls = STATS_DOWN;
            L.prefetch = l + 1 < c.n_layers ? m->layers[l + 1].attn_norm : m->out_norm; L.prefetch_bytes = (size_t)c.dim * 4;
            if (l + 1 < c.n_layers) {
                const slai_qmatrix* nx[3] = {m->layers[l + 1].wq, m->layers[l + 1].wk, m->layers[l + 1].wv};
                L.ahead = plan_ahead(nx, 3, 0, cap);
            } else {
                L.ahead = plan_ahead1(m->output ? m->output : m->embd_q, 0, cap);
            }
            if ((rc = row_parallel(L))) return rc;
        }
    }
    // logits = Wout rmsnorm(x)                                                  transformer.rs:368-375
    const slai_qmatrix* wout = m->output ? m->output : (m->embd_q ? m->embd_q : &m->embd_as_matrix);
    if (wout->fmt == SLAI_FMT_F32) {
        if ((rc = slai_rms_norm(ctx, m->xb, m->x, m->out_norm, c.dim, c.rms_norm_eps))) return rc;
        n++;
        GemvLaunch L;
        L.fmt = SLAI_FMT_F32; L.K = c.dim; L.nseg = 1; L.seg[0] = seg_of(wout, 0, c.vocab_size, nullptr, 0, 0);
        L.v = m->xb; L.out = m->logits; L.pdl = false;
        if ((rc = gemv_launch(ctx, L))) return rc;
        n++;
    } else {
        GemvLaunch L;
        const int vrows = m->out_sharded ? c.vocab_size / m->tp : c.vocab_size;
        L.fmt = wout->fmt; L.K = c.dim; L.nseg = 1; L.seg[0] = seg_of(wout, 0, vrows, nullptr, 0, 0);
        L.v = m->x; L.out = m->out_sharded ? m->logits_part : m->logits; L.pro = PRO_RMS; L.norm_w = m->out_norm; L.eps = c.rms_norm_eps;
        L.epi = EPI_STORE;
        L.pdl = pdl;
        L.stats_cls = STATS_LOGITS;
        {   // the next token starts with layer 0's q / k / v again
            const slai_qmatrix* nx[3] = {m->layers[0].wq, m->layers[0].wk, m->layers[0].wv};
            L.ahead = plan_ahead(nx, 3, 0, ahead_cap_bytes());
        }
        consume_exchange(L);
        if ((rc = gemv_launch(ctx, L))) return rc;
        n++;
        if (m->out_sharded) {  // every rank's slice of the logits, in rank order = vocabulary order
            if ((rc = tp_all_gather(ctx, m->logits_part, m->logits, vrows))) return rc;
            n++;
        }
    }
    if (kind == G_SAMPLED) rc = launch_sample(ctx, m->logits, c.vocab_size, m->d_samp, m->sc.d + 2, 0.f, false, m->d_samp_scratch, m->sc.d + 3, pdl);
    else rc = launch_argmax(ctx, m->logits, c.vocab_size, m->sc.d + 3, pdl);
    if (rc) return rc;
    n++;
    if (kind == G_GENERATE || kind == G_SAMPLED) {
        if ((rc = launch_advance(ctx, d_token, d_pos, m->sc.d + 3, m->d_history, c.vocab_size, pdl))) return rc;
        n++;
    } else if (kind == G_FORCED) {
        // next token comes from the prompt: history[] holds tokens[1..]; advance copies history[step]
        if ((rc = launch_advance(ctx, d_token, d_pos, nullptr, m->d_history, c.vocab_size, pdl))) return rc;
        n++;
    }
    m->launches = n;
    return SLAI_OK;
}


template <class M, class RecordFn>
static int run_graph(M* m, int kind, RecordFn record) {
    slai_ctx* ctx = m->ctx;
    if (!m->graphs.use_graph) return record(m, kind);
    if (!m->graphs.warmed[kind]) {
        m->graphs.warmed[kind] = true;
        return record(m, kind);
    }
    if (!m->graphs.exec[kind]) {
        cudaGraph_t graph = nullptr;
        SLAI_CHECK_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        int rc = record(m, kind);
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
        if (rc == SLAI_OK && e == cudaSuccess) {
            e = cudaGraphInstantiate(&m->graphs.exec[kind], graph, 0);
            if (e != cudaSuccess) m->graphs.exec[kind] = nullptr;
        }
        if (graph) cudaGraphDestroy(graph);
        if (rc != SLAI_OK || e != cudaSuccess) {
            // some launches (e.g. cooperative ones on older drivers) cannot be captured: run eagerly from now on
            fprintf(stderr, "slai_b200: CUDA graph capture of the decode step failed (%s); launching eagerly\n",
                    e != cudaSuccess ? cudaGetErrorString(e) : "record error");
            cudaGetLastError();
            m->graphs.use_graph = false;
            return record(m, kind);
        }
    }
    SLAI_CHECK_CUDA(ctx, cudaGraphLaunch(m->graphs.exec[kind], ctx->stream));
    return SLAI_OK;
}

SLAI_API int slai_llama_create(slai_ctx* ctx, const slai_llama_config* cfg, slai_llama** out) {
    if (!ctx || !cfg || !out) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    *out = nullptr;
    const slai_llama_config& c = *cfg;
    SLAI_REQUIRE(ctx, c.dim > 0 && c.hidden_dim > 0 && c.n_layers > 0 && c.n_q_heads > 0 && c.n_kv_heads > 0 && c.vocab_size > 0 &&
                          c.seq_len > 0, SLAI_ERR_INVALID_ARG, "llama: non-positive dimension");
    SLAI_REQUIRE(ctx, c.dim % c.n_q_heads == 0 && c.n_q_heads % c.n_kv_heads == 0, SLAI_ERR_SHAPE, "llama: head counts do not divide");
    SLAI_REQUIRE(ctx, (c.dim / c.n_q_heads) % 2 == 0, SLAI_ERR_SHAPE, "llama: odd head size");
    SLAI_REQUIRE(ctx, c.kv_dtype == SLAI_KV_F16 || c.kv_dtype == SLAI_KV_F32, SLAI_ERR_INVALID_ARG, "llama: unknown kv_dtype");
    const int tp = c.tp_size > 1 ? c.tp_size : 1;
    if (tp > 1) {  // (checked before anything is allocated)
        SLAI_REQUIRE(ctx, ctx->tp_comm && ctx->tp_size == c.tp_size && ctx->tp_rank == c.tp_rank, SLAI_ERR_INVALID_ARG,
                     "llama: tp_rank/tp_size %d/%d do not match the context's group (slai_tp_init)", c.tp_rank, c.tp_size);
        SLAI_REQUIRE(ctx, c.n_kv_heads % tp == 0 && c.hidden_dim % tp == 0 && (c.hidden_dim / tp) % 16 == 0, SLAI_ERR_SHAPE,
                     "llama: %d KV heads / hidden %d do not split over %d ranks", c.n_kv_heads, c.hidden_dim, tp);
    }
    slai_llama* m = new slai_llama();
    m->ctx = ctx;
    m->cfg = c;
    // derived sizes: Llama2Config::derived_configs (models/llama2/cpu.rs:111-143)
    m->tp = tp;
    m->head_size = c.dim / c.n_q_heads;
    m->kv_mul = c.n_q_heads / c.n_kv_heads;
    m->n_q_local = c.n_q_heads / m->tp;
    m->q_dim = m->n_q_local * m->head_size;
    m->kv_dim = c.n_kv_heads / m->tp * m->head_size;
    m->hidden = c.hidden_dim / m->tp;
    m->layers.resize(c.n_layers);
    const size_t esz = c.kv_dtype == SLAI_KV_F16 ? 2 : 4;
    m->kv_layer_elems = (size_t)c.seq_len * m->kv_dim;
    const char* ng = getenv("SLAI_NO_GRAPH");
    m->graphs.use_graph = !(ng && ng[0] == '1');
    m->history_cap = c.seq_len + 8;
    m->attn_scratch_bytes = attention_scratch_bytes(ctx, m->n_q_local, m->kv_mul, m->head_size, c.seq_len - 1);
    bool ok = cudaMalloc(&m->x, (size_t)c.dim * 4) == cudaSuccess && cudaMalloc(&m->xb, (size_t)c.dim * 4) == cudaSuccess &&
              cudaMalloc(&m->xpart, (size_t)c.dim * 4) == cudaSuccess && cudaMalloc(&m->rope_cs, 2 * 256 * 4) == cudaSuccess &&
              cudaMalloc(&m->q, (size_t)c.dim * 4) == cudaSuccess && cudaMalloc(&m->hb, (size_t)c.hidden_dim * 4) == cudaSuccess &&
              cudaMalloc(&m->hb2, (size_t)c.hidden_dim * 4) == cudaSuccess &&
              cudaMalloc(&m->ktmp, (size_t)c.dim * 4) == cudaSuccess && cudaMalloc(&m->vtmp, (size_t)c.dim * 4) == cudaSuccess &&
              cudaMalloc(&m->logits, (size_t)c.vocab_size * 4) == cudaSuccess &&
              cudaMalloc(&m->kcache, m->kv_layer_elems * c.n_layers * esz) == cudaSuccess &&
              cudaMalloc(&m->vcache, m->kv_layer_elems * c.n_layers * esz) == cudaSuccess &&
              cudaMalloc(&m->sc.d, 64) == cudaSuccess && cudaMalloc(&m->d_history, (size_t)m->history_cap * 4) == cudaSuccess &&
              cudaMalloc(&m->attn_scratch, m->attn_scratch_bytes) == cudaSuccess;
    if (ok) {
        ok = cudaMemsetAsync(m->kcache, 0, m->kv_layer_elems * c.n_layers * esz, ctx->stream) == cudaSuccess &&
             cudaMemsetAsync(m->vcache, 0, m->kv_layer_elems * c.n_layers * esz, ctx->stream) == cudaSuccess &&
             cudaMemsetAsync(m->sc.d, 0, 64, ctx->stream) == cudaSuccess &&
             cudaMemsetAsync(m->d_history, 0, (size_t)m->history_cap * 4, ctx->stream) == cudaSuccess;
    }
    m->rope_theta = rope_table(ctx, m->head_size, c.rope_base_freq);
    if (!ok || !m->rope_theta) {
        cudaGetLastError();
        slai_llama_destroy(m);
        return slai_set_error(ctx, SLAI_ERR_OOM, "llama: cannot allocate the model state");
    }
    *out = m;
    return SLAI_OK;
}

// ---- several sequences decoded together ------------------------------------------------------------------------------
// Every sequence has its own KV cache and position; one step takes one token of each and reads every weight matrix once
// for all of them (the batched GEMV, gemv_batch.cu).  Per layer: RmsNorm of all rows, q / k / v products, then per sequence
// RoPE + cache write and the single-query attention kernel on that sequence's cache, output product + residual, RmsNorm,
// gate / up products, SiLU, down product + residual (the operator sequence of transformer.rs:327-365 on `n_seq` columns).
SLAI_API int slai_llama_batch_reserve(slai_llama* m, int32_t n_seq) {
    if (!m) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    slai_ctx* ctx = m->ctx;
    const slai_llama_config& c = m->cfg;
    SLAI_REQUIRE(ctx, n_seq >= 0 && n_seq <= 8, SLAI_ERR_INVALID_ARG, "batch: %d sequences (0..8)", n_seq);
    SLAI_REQUIRE(ctx, m->tp == 1, SLAI_ERR_INVALID_ARG, "batch: sharded models decode one sequence at a time");
    llama_drop_batch(m);
    if (n_seq == 0) return SLAI_OK;
    const size_t esz = c.kv_dtype == SLAI_KV_F16 ? 2 : 4;
    m->bt_cache_bytes = (size_t)c.n_layers * m->kv_layer_elems * esz;
    const size_t B = (size_t)n_seq;
    const size_t wide = (size_t)std::max(c.dim, m->q_dim);
    bool ok = cudaMalloc(&m->bt_k, B * m->bt_cache_bytes) == cudaSuccess && cudaMalloc(&m->bt_v, B * m->bt_cache_bytes) == cudaSuccess &&
              cudaMalloc(&m->bt_x, B * c.dim * 4) == cudaSuccess && cudaMalloc(&m->bt_xn, B * wide * 4) == cudaSuccess &&
              cudaMalloc(&m->bt_q, B * m->q_dim * 4) == cudaSuccess && cudaMalloc(&m->bt_qkv, B * (m->q_dim + 2 * m->kv_dim) * 4) == cudaSuccess &&
              cudaMalloc(&m->bt_xb, B * m->q_dim * 4) == cudaSuccess &&
              cudaMalloc(&m->bt_t, B * c.dim * 4) == cudaSuccess && cudaMalloc(&m->bt_g, B * m->hidden * 4) == cudaSuccess &&
              cudaMalloc(&m->bt_u, B * m->hidden * 4) == cudaSuccess && cudaMalloc(&m->bt_logits, B * c.vocab_size * 4) == cudaSuccess &&
              cudaMalloc(&m->bt_i, 24 * sizeof(int)) == cudaSuccess && cudaMalloc(&m->bt_attn, B * m->attn_scratch_bytes) == cudaSuccess &&
              cudaMalloc(&m->bt_tickets, B * 1024 * sizeof(unsigned int)) == cudaSuccess;
    if (ok)
        ok = cudaMemsetAsync(m->bt_k, 0, B * m->bt_cache_bytes, ctx->stream) == cudaSuccess &&
             cudaMemsetAsync(m->bt_v, 0, B * m->bt_cache_bytes, ctx->stream) == cudaSuccess &&
             cudaMemsetAsync(m->bt_xb, 0, B * m->q_dim * 4, ctx->stream) == cudaSuccess &&
             cudaMemsetAsync(m->bt_tickets, 0, B * 1024 * sizeof(unsigned int), ctx->stream) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        m->bt_n = 1;  // so that the buffers obtained so far are released
        llama_drop_batch(m);
        return slai_set_error(ctx, SLAI_ERR_OOM, "batch: cannot allocate caches and activations for %d sequences", n_seq);
    }
    m->bt_n = n_seq;
    return SLAI_OK;
}

// One token of every sequence b < n_seq at position h_pos[b] (a negative position leaves sequence b out of this step: its
// cache is not touched and its outputs mean nothing).  h_logits: n_seq x vocab floats or null; h_next: the greedy choice
// per sequence or null.
// The launches of one step of B sequences (tokens and positions are in bt_i); attention is sized for contexts of up to
// `cap_pos` + 1 positions.
static int llama_batch_record(slai_llama* m, int B, int cap_pos) {
    slai_ctx* ctx = m->ctx;
    const slai_llama_config& c = m->cfg;
    int* d_tok = m->bt_i;
    int* d_pos = m->bt_i + 8;
    int* d_next = m->bt_i + 16;
    int rc;
    if ((rc = prefill_embed_launch(ctx, m->bt_x, c.dim, d_tok, B, m->embd_q ? nullptr : m->token_embd, m->embd_q))) return rc;
    const size_t esz = c.kv_dtype == SLAI_KV_F16 ? 2 : 4;
    const long long kv_head_stride = (long long)c.seq_len * m->head_size;
    const int qkv_ld = m->q_dim + 2 * m->kv_dim;
    // out[b * ldo + r] (=, +=) (W in[b])[r]: one pass over a quantised matrix for all sequences (the residual add or the SiLU
    // gate folded into its store), else vector by vector and the operators after it
    auto product = [&](const slai_qmatrix* wm, const float* in, float* out, long long ldo, int epi = BATCH_STORE, float* gate = nullptr) -> int {
        if (B > 1 && gemv_batch_supported(wm)) return gemv_batch_launch(ctx, out, wm, in, B, ldo, epi, gate);
        float* dst = epi == BATCH_ADD ? m->bt_t : out;  // (the residual streams are dense: ldo == rows)
        for (int b = 0; b < B; b++) {
            const int r = slai_gemv_quant(ctx, dst + (size_t)b * ldo, wm, in + (size_t)b * wm->ncols, 1);
            if (r) return r;
        }
        if (epi == BATCH_ADD) return slai_add_assign(ctx, out, m->bt_t, (int64_t)B * ldo);
        if (epi == BATCH_SILU) {
            int r = slai_silu_gate(ctx, gate, out, (int64_t)B * ldo);
            if (!r) r = slai_copy(ctx, out, gate, (int64_t)B * ldo);
            return r;
        }
        return SLAI_OK;
    };
    for (int l = 0; l < c.n_layers; l++) {
        const LlamaLayer& w = m->layers[l];
        void* kc = (char*)m->bt_k + (size_t)l * m->kv_layer_elems * esz;  // layer l of sequence 0; sequence b is bt_cache_bytes further
        void* vc = (char*)m->bt_v + (size_t)l * m->kv_layer_elems * esz;
        if ((rc = rms_norm_rows_launch(ctx, m->bt_xn, m->bt_x, w.attn_norm, c.dim, B, c.rms_norm_eps))) return rc;
        // q, k, v in one launch where the three matrices can be walked as one (same format, heights multiples of 16)
        const bool qkv_one = B > 1 && gemv_batch_supported(w.wq) && w.wk->fmt == w.wq->fmt && w.wv->fmt == w.wq->fmt && m->q_dim % 16 == 0 &&
                             m->kv_dim % 16 == 0;
        if (qkv_one) {
            const slai_qmatrix* ws[3] = {w.wq, w.wk, w.wv};
            if ((rc = gemv_batch_launch_multi(ctx, m->bt_qkv, ws, 3, m->bt_xn, B, qkv_ld, BATCH_STORE, nullptr))) return rc;
        } else {
            if ((rc = product(w.wq, m->bt_xn, m->bt_qkv, qkv_ld))) return rc;
            if ((rc = product(w.wk, m->bt_xn, m->bt_qkv + m->q_dim, qkv_ld))) return rc;
            if ((rc = product(w.wv, m->bt_xn, m->bt_qkv + m->q_dim + m->kv_dim, qkv_ld))) return rc;
        }
        if ((rc = rope_kv_store_seqs_launch(ctx, m->bt_qkv, qkv_ld, m->q_dim, m->kv_dim, m->head_size, d_pos, B, m->rope_theta, c.rope_variant != 0,
                                            m->bt_q, kc, vc, c.kv_dtype == SLAI_KV_F16, kv_head_stride, (long long)m->bt_cache_bytes)))
            return rc;
        {
            AttnLaunch A = {};
            A.q = m->bt_q; A.kcache = kc; A.vcache = vc; A.kv_dtype = c.kv_dtype;
            A.pos_stride = m->head_size; A.head_stride = kv_head_stride;
            A.n_heads = m->n_q_local; A.kv_mul = m->kv_mul; A.head_size = m->head_size;
            A.d_pos = nullptr; A.max_pos = cap_pos; A.out = m->bt_xb; A.pdl = false;
            A.scratch = m->bt_attn; A.scratch_bytes = (size_t)m->bt_n * m->attn_scratch_bytes;
            A.batch = B; A.pos0 = 0; A.q_batch_stride = m->q_dim; A.out_batch_stride = m->q_dim; A.batch_counters = m->bt_tickets;
            A.cache_batch_stride = (long long)m->bt_cache_bytes; A.d_pos_batch = d_pos;
            if ((rc = attention_launch(ctx, A))) return rc;
        }
        if ((rc = product(w.wo, m->bt_xb, m->bt_x, c.dim, BATCH_ADD))) return rc;
        if ((rc = rms_norm_rows_launch(ctx, m->bt_xn, m->bt_x, w.ffn_norm, c.dim, B, c.rms_norm_eps))) return rc;
        if (B > 1 && gemv_batch_supported(w.wgate) && w.wup->fmt == w.wgate->fmt && m->hidden % 16 == 0) {
            const slai_qmatrix* ws[2] = {w.wgate, w.wup};  // gate and up in one launch, SiLU in its store
            if ((rc = gemv_batch_launch_multi(ctx, m->bt_u, ws, 2, m->bt_xn, B, m->hidden, BATCH_PAIR_SILU, nullptr))) return rc;
        } else {
            if ((rc = product(w.wgate, m->bt_xn, m->bt_g, m->hidden))) return rc;
            if ((rc = product(w.wup, m->bt_xn, m->bt_u, m->hidden, BATCH_SILU, m->bt_g))) return rc;
        }
        if ((rc = product(w.wdown, m->bt_u, m->bt_x, c.dim, BATCH_ADD))) return rc;
    }
    const slai_qmatrix* wout = m->output ? m->output : (m->embd_q ? m->embd_q : &m->embd_as_matrix);
    if ((rc = rms_norm_rows_launch(ctx, m->bt_xn, m->bt_x, m->out_norm, c.dim, B, c.rms_norm_eps))) return rc;
    if ((rc = product(wout, m->bt_xn, m->bt_logits, c.vocab_size))) return rc;
    for (int b = 0; b < B; b++)
        if ((rc = launch_argmax(ctx, m->bt_logits + (size_t)b * c.vocab_size, c.vocab_size, d_next + b, false))) return rc;
    return SLAI_OK;
}

// One token of every sequence b < n_seq at position h_pos[b] (a negative position leaves sequence b out of this step: its
// cache is not touched and its outputs mean nothing).  h_logits: n_seq x vocab floats or null; h_next: the greedy choice
// per sequence or null.  The first step of a batch size runs launch by launch; later ones replay a graph of the step, captured
// again whenever the longest context crosses a multiple of 256 positions (the attention launch is sized for the context).
SLAI_API int slai_llama_decode_batch(slai_llama* m, int32_t n_seq, const int32_t* h_tokens, const int32_t* h_pos, float* h_logits,
                                     int32_t* h_next) {
    if (!m || !h_tokens || !h_pos) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    slai_ctx* ctx = m->ctx;
    const slai_llama_config& c = m->cfg;
    SLAI_REQUIRE(ctx, n_seq >= 1 && n_seq <= m->bt_n, SLAI_ERR_INVALID_ARG, "batch: %d sequences, %d reserved (slai_llama_batch_reserve)", n_seq, m->bt_n);
    SLAI_REQUIRE(ctx, m->out_norm && (m->token_embd || m->embd_q), SLAI_ERR_INVALID_ARG, "llama: embedding / output norm not set");
    int h[24] = {};
    int max_pos = 0;
    for (int b = 0; b < n_seq; b++) {
        SLAI_REQUIRE(ctx, h_pos[b] < c.seq_len, SLAI_ERR_INVALID_ARG, "batch: position %d of sequence %d exceeds the context", h_pos[b], b);
        SLAI_REQUIRE(ctx, h_pos[b] < 0 || (h_tokens[b] >= 0 && h_tokens[b] < c.vocab_size), SLAI_ERR_INVALID_ARG, "batch: token %d out of range",
                     h_tokens[b]);
        h[b] = h_pos[b] < 0 ? 0 : h_tokens[b];
        h[8 + b] = h_pos[b] < 0 ? -1 : h_pos[b];
        max_pos = std::max(max_pos, (int)h_pos[b]);
    }
    for (auto& w : m->layers) {
        SLAI_REQUIRE(ctx, w.wq && w.wk && w.wv && w.wo && w.wgate && w.wup && w.wdown && w.attn_norm && w.ffn_norm, SLAI_ERR_INVALID_ARG,
                     "llama: a layer's weights are not set");
        SLAI_REQUIRE(ctx, !w.bq && !w.bk && !w.bv, SLAI_ERR_UNSUPPORTED_FORMAT, "batch: q / k / v biases are not supported");
    }
    SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(m->bt_i, h, sizeof(h), cudaMemcpyHostToDevice, ctx->stream));
    const int B = n_seq;
    const int cap_pos = std::min(c.seq_len - 1, (max_pos / 256 + 1) * 256 - 1);
    int rc = SLAI_OK;
    if (!m->graphs.use_graph || !m->bt_warm[B]) {
        m->bt_warm[B] = true;  // the first step also sets kernel attributes and sizes the scratch: not inside a capture
        rc = llama_batch_record(m, B, cap_pos);
    } else {
        if (m->bt_exec[B] && m->bt_cap[B] != cap_pos) {
            cudaGraphExecDestroy(m->bt_exec[B]);
            m->bt_exec[B] = nullptr;
        }
        if (!m->bt_exec[B]) {
            cudaGraph_t graph = nullptr;
            SLAI_CHECK_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
            rc = llama_batch_record(m, B, cap_pos);
            cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
            if (rc == SLAI_OK && e == cudaSuccess) {
                e = cudaGraphInstantiate(&m->bt_exec[B], graph, 0);
                if (e != cudaSuccess) m->bt_exec[B] = nullptr;
            }
            if (graph) cudaGraphDestroy(graph);
            if (rc != SLAI_OK || e != cudaSuccess) {
                cudaGetLastError();
                m->bt_exec[B] = nullptr;
                m->graphs.use_graph = false;  // launch by launch from now on
                rc = llama_batch_record(m, B, cap_pos);
            } else {
                m->bt_cap[B] = cap_pos;
            }
        }
        if (m->bt_exec[B]) {
            SLAI_CHECK_CUDA(ctx, cudaGraphLaunch(m->bt_exec[B], ctx->stream));
            rc = SLAI_OK;
        }
    }
    if (rc) return rc;
    int* d_next = m->bt_i + 16;
    if (h_logits) SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(h_logits, m->bt_logits, (size_t)B * c.vocab_size * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (h_next) SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(h_next, d_next, (size_t)B * 4, cudaMemcpyDeviceToHost, ctx->stream));
    SLAI_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return slai_check_wait_flag(ctx);
}

SLAI_API int slai_llama_destroy(slai_llama* m) {
    if (!m) return SLAI_OK;
    SLAI_ENTER(m->ctx);
    cudaStreamSynchronize(m->ctx->stream);
    destroy_graphs(m->graphs);
    llama_drop_prefill(m);
    llama_drop_batch(m);
    for (auto& l : m->layers) {
        cudaFree(l.attn_norm); cudaFree(l.ffn_norm); cudaFree(l.bq); cudaFree(l.bk); cudaFree(l.bv);
    }
    cudaFree(m->token_embd); cudaFree(m->out_norm);
    cudaFree(m->x); cudaFree(m->xb); cudaFree(m->xpart); cudaFree(m->q); cudaFree(m->hb); cudaFree(m->hb2); cudaFree(m->logits);
    cudaFree(m->logits_part); cudaFree(m->ktmp); cudaFree(m->vtmp);
    cudaFree(m->kcache); cudaFree(m->vcache); cudaFree(m->sc.d); cudaFree(m->d_history); cudaFree(m->attn_scratch);
    cudaFree(m->d_samp); cudaFree(m->d_samp_scratch); cudaFree(m->rope_cs);
    delete m;
    return SLAI_OK;
}

SLAI_API int slai_llama_set_matrix(slai_llama* m, int id, int layer, const slai_qmatrix* w) {
    if (!m || !w) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    slai_ctx* ctx = m->ctx;
    const slai_llama_config& c = m->cfg;
    destroy_graphs(m->graphs);
    llama_drop_batch_graphs(m);
    auto shape_is = [&](int64_t r, int64_t k) { return w->nrows == r && w->ncols == k; };
    if (id == SLAI_W_OUTPUT) {
        // tensor parallel: either the whole matrix on every rank, or this rank's vocab / tp consecutive rows (the
        // logits are then gathered from all ranks after the product)
        const bool part = m->tp > 1 && c.vocab_size % (16 * m->tp) == 0 && shape_is(c.vocab_size / m->tp, c.dim);
        SLAI_REQUIRE(ctx, part || shape_is(c.vocab_size, c.dim), SLAI_ERR_SHAPE, "llama: output matrix must be vocab x dim%s",
                     m->tp > 1 ? " (or vocab / tp x dim, vocab / tp a multiple of 16)" : "");
        if (part && !m->logits_part) SLAI_CHECK_CUDA(ctx, cudaMalloc(&m->logits_part, (size_t)c.vocab_size / m->tp * 4));
        m->out_sharded = part;
        m->output = w;
        return SLAI_OK;
    }
    if (id == SLAI_W_TOKEN_EMBD) {
        SLAI_REQUIRE(ctx, shape_is(c.vocab_size, c.dim), SLAI_ERR_SHAPE, "llama: token_embd must be vocab x dim");
        m->embd_q = w;
        return SLAI_OK;
    }
    SLAI_REQUIRE(ctx, layer >= 0 && layer < c.n_layers, SLAI_ERR_INVALID_ARG, "llama: layer %d out of range", layer);
    LlamaLayer& l = m->layers[layer];
    switch (id) {
        case SLAI_W_Q: SLAI_REQUIRE(ctx, shape_is(m->q_dim, c.dim), SLAI_ERR_SHAPE, "llama: attn_q must be (dim / tp) x dim"); l.wq = w; break;
        case SLAI_W_K: SLAI_REQUIRE(ctx, shape_is(m->kv_dim, c.dim), SLAI_ERR_SHAPE, "llama: attn_k must be kv_dim x dim"); l.wk = w; break;
        case SLAI_W_V: SLAI_REQUIRE(ctx, shape_is(m->kv_dim, c.dim), SLAI_ERR_SHAPE, "llama: attn_v must be kv_dim x dim"); l.wv = w; break;
        case SLAI_W_O: SLAI_REQUIRE(ctx, shape_is(c.dim, m->q_dim), SLAI_ERR_SHAPE, "llama: attn_output must be dim x (dim / tp)"); l.wo = w; break;
        case SLAI_W_GATE: SLAI_REQUIRE(ctx, shape_is(m->hidden, c.dim), SLAI_ERR_SHAPE, "llama: ffn_gate must be (hidden / tp) x dim"); l.wgate = w; break;
        case SLAI_W_UP: SLAI_REQUIRE(ctx, shape_is(m->hidden, c.dim), SLAI_ERR_SHAPE, "llama: ffn_up must be (hidden / tp) x dim"); l.wup = w; break;
        case SLAI_W_DOWN: SLAI_REQUIRE(ctx, shape_is(c.dim, m->hidden), SLAI_ERR_SHAPE, "llama: ffn_down must be dim x (hidden / tp)"); l.wdown = w; break;
        default: return slai_set_error(ctx, SLAI_ERR_INVALID_ARG, "llama: weight id %d is not a matrix", id);
    }
    return SLAI_OK;
}

static int llama_set_f32_impl(slai_llama* m, int id, int layer, const float* data, int64_t n, bool dev) {
    if (!m || !data) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    slai_ctx* ctx = m->ctx;
    const slai_llama_config& c = m->cfg;
    destroy_graphs(m->graphs);
    llama_drop_batch_graphs(m);
    if (id == SLAI_W_TOKEN_EMBD) {
        SLAI_REQUIRE(ctx, n == (int64_t)c.vocab_size * c.dim, SLAI_ERR_SHAPE, "llama: token_embd needs vocab*dim floats");
        int rc = copy_f32(ctx, &m->token_embd, data, n, dev);
        if (rc) return rc;
        m->embd_as_matrix.ctx = ctx; m->embd_as_matrix.fmt = SLAI_FMT_F32; m->embd_as_matrix.nrows = c.vocab_size;
        m->embd_as_matrix.ncols = c.dim; m->embd_as_matrix.tile_bytes = (int64_t)c.dim * 4;
        m->embd_as_matrix.data = (uint8_t*)m->token_embd; m->embd_as_matrix.owns = false;
        return SLAI_OK;
    }
    if (id == SLAI_W_OUT_NORM) {
        SLAI_REQUIRE(ctx, n == c.dim, SLAI_ERR_SHAPE, "llama: output_norm needs dim floats");
        return copy_f32(ctx, &m->out_norm, data, n, dev);
    }
    SLAI_REQUIRE(ctx, layer >= 0 && layer < c.n_layers, SLAI_ERR_INVALID_ARG, "llama: layer %d out of range", layer);
    LlamaLayer& l = m->layers[layer];
    float** dst = nullptr;
    int64_t want = c.dim;
    switch (id) {
        case SLAI_W_ATTN_NORM: dst = &l.attn_norm; break;
        case SLAI_W_FFN_NORM: dst = &l.ffn_norm; break;
        case SLAI_W_BQ: dst = &l.bq; want = m->q_dim; break;
        case SLAI_W_BK: dst = &l.bk; want = m->kv_dim; break;
        case SLAI_W_BV: dst = &l.bv; want = m->kv_dim; break;
        default: return slai_set_error(ctx, SLAI_ERR_INVALID_ARG, "llama: weight id %d is not an f32 vector", id);
    }
    SLAI_REQUIRE(ctx, n == want, SLAI_ERR_SHAPE, "llama: weight %d needs %lld floats, got %lld", id, (long long)want, (long long)n);
    return copy_f32(ctx, dst, data, n, dev);
}
SLAI_API int slai_llama_set_f32(slai_llama* m, int id, int layer, const float* h_data, int64_t n) {
    return llama_set_f32_impl(m, id, layer, h_data, n, false);
}
SLAI_API int slai_llama_set_f32_device(slai_llama* m, int id, int layer, const float* d_data, int64_t n) {
    return llama_set_f32_impl(m, id, layer, d_data, n, true);
}

template <class M>
static int set_scalars(M* m, int token, int pos, int step) {
    const int h[4] = {token, pos, step, 0};
    SLAI_CHECK_CUDA(m->ctx, cudaMemcpyAsync(m->sc.d, h, sizeof(h), cudaMemcpyHostToDevice, m->ctx->stream));
    return SLAI_OK;
}

template <class M, class RecordFn>
static int decode_impl(M* m, RecordFn record, int vocab, int seq_len, int32_t token, int32_t pos, float* h_logits,
                       int32_t* next_token) {
    slai_ctx* ctx = m->ctx;
    SLAI_REQUIRE(ctx, token >= 0 && token < vocab, SLAI_ERR_INVALID_ARG, "decode: token %d out of range", token);
    SLAI_REQUIRE(ctx, pos >= 0 && pos < seq_len, SLAI_ERR_INVALID_ARG, "decode: pos %d out of range", pos);
    int rc = set_scalars(m, token, pos, 0);
    if (rc) return rc;
    if ((rc = run_graph(m, G_DECODE, record))) return rc;
    if (h_logits) SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(h_logits, m->logits, (size_t)vocab * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (next_token) SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(next_token, m->sc.d + 3, 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (h_logits || next_token) {
        SLAI_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        return slai_check_wait_flag(ctx);  // a step whose bounded wait ran out must not hand out its token
    }
    return SLAI_OK;
}

template <class M, class RecordFn>
static int generate_impl(M* m, RecordFn record, int vocab, int seq_len, int32_t token, int32_t pos, int32_t n, int32_t* h_tokens,
                         int kind = G_GENERATE) {
    slai_ctx* ctx = m->ctx;
    SLAI_REQUIRE(ctx, token >= 0 && token < vocab, SLAI_ERR_INVALID_ARG, "generate: token %d out of range", token);
    SLAI_REQUIRE(ctx, n > 0 && pos >= 0 && pos + n <= seq_len && n <= m->history_cap, SLAI_ERR_INVALID_ARG,
                 "generate: positions %d..%d exceed the context", pos, pos + n);
    int rc = set_scalars(m, token, pos, 0);
    if (rc) return rc;
    for (int i = 0; i < n; i++)
        if ((rc = run_graph(m, kind, record))) return rc;
    if (h_tokens) SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(h_tokens, m->d_history, (size_t)n * 4, cudaMemcpyDeviceToHost, ctx->stream));
    SLAI_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return slai_check_wait_flag(ctx);
}

template <class M, class RecordFn>
static int prefill_impl(M* m, RecordFn record, int vocab, int seq_len, const int32_t* h_tokens, int32_t n, int32_t pos0,
                        float* h_last_logits) {
    slai_ctx* ctx = m->ctx;
    SLAI_REQUIRE(ctx, h_tokens && n > 0 && pos0 >= 0 && pos0 + n <= seq_len && n < m->history_cap, SLAI_ERR_INVALID_ARG,
                 "prefill: positions %d..%d exceed the context", pos0, pos0 + n);
    for (int i = 0; i < n; i++)
        SLAI_REQUIRE(ctx, h_tokens[i] >= 0 && h_tokens[i] < vocab, SLAI_ERR_INVALID_ARG, "prefill: token %d out of range", h_tokens[i]);
    // history[step] = the token to feed after step `step` (tokens[1..]; the entry after the last is unused)
    std::vector<int32_t> next(n, 0);
    for (int i = 0; i + 1 < n; i++) next[i] = h_tokens[i + 1];
    SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(m->d_history, next.data(), (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
    int rc = set_scalars(m, h_tokens[0], pos0, 0);
    if (rc) return rc;
    SLAI_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // `next` leaves scope
    for (int i = 0; i < n; i++)
        if ((rc = run_graph(m, G_FORCED, record))) return rc;
    if (h_last_logits) SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(h_last_logits, m->logits, (size_t)vocab * 4, cudaMemcpyDeviceToHost, ctx->stream));
    SLAI_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return slai_check_wait_flag(ctx);
}

// ---- prompt processing as GEMMs -----------------------------------------------------------------------------------------
// The T prompt tokens go through every layer together (prefill.cu): per layer RmsNorm + fp16-pair split, q / k / v
// GEMMs, RoPE + KV-cache write, causal attention (a tiled kernel of its own, 16 query tokens per CTA), output GEMM
// with residual, RmsNorm + split, gate and up GEMMs, SiLU + split, down GEMM with residual.  Only the last token's
// logits are needed: its row of the residual stream goes back into the decode state and the decode step's own final
// norm + logits GEMV (+ greedy choice) run on it.  Sharded models run the same sequence on their shards; the two
// row-parallel products of a layer (output and down projection) leave a partial [tokens][dim] on every rank, summed with
// one all-reduce each and added to the residual stream, which stays identical on all ranks.
static bool llama_prefill_eligible(const slai_llama* m, int n) {
    const char* e = getenv("SLAI_PREFILL_SEQUENTIAL");
    if (e && e[0] == '1') return false;
    if (n < 16 || m->kv_mul > 8) return false;
    if (m->tp > 1 && !m->ctx->tp_comm) return false;  // the partial products of a sharded model are summed with the group's all-reduce
    if (!m->out_norm || (!m->token_embd && !m->embd_q)) return false;
    for (auto& w : m->layers) {
        const slai_qmatrix* ms[7] = {w.wq, w.wk, w.wv, w.wo, w.wgate, w.wup, w.wdown};
        for (auto* q : ms)
            if (!q || q->fmt == SLAI_FMT_F32 || q->ncols % 64 != 0) return false;
        if (!w.attn_norm || !w.ffn_norm) return false;
    }
    return true;
}

static int llama_prefill_reserve(slai_llama* m, int t_pad, int attn_batch, size_t attn_bytes, int n_kv) {
    slai_ctx* ctx = m->ctx;
    const slai_llama_config& c = m->cfg;
    if (t_pad > m->pf_cap || attn_batch > m->pf_attn_batch) llama_drop_prefill(m);
    if (!m->pf_cap) {
        const size_t T = (size_t)t_pad;
        const size_t kmax = (size_t)std::max(std::max(c.dim, m->hidden), m->q_dim);
        bool ok = cudaMalloc(&m->pf_x, T * c.dim * 4) == cudaSuccess && cudaMalloc(&m->pf_qkv, T * (m->q_dim + 2 * m->kv_dim) * 4) == cudaSuccess &&
                  cudaMalloc(&m->pf_q, T * m->q_dim * 4) == cudaSuccess && cudaMalloc(&m->pf_xb, T * m->q_dim * 4) == cudaSuccess &&
                  cudaMalloc(&m->pf_g, T * m->hidden * 4) == cudaSuccess && cudaMalloc(&m->pf_u, T * m->hidden * 4) == cudaSuccess &&
                  (m->tp == 1 || cudaMalloc(&m->pf_part, T * c.dim * 4) == cudaSuccess) &&
                  cudaMalloc(&m->pf_hi, T * kmax * 2) == cudaSuccess && cudaMalloc(&m->pf_lo, T * kmax * 2) == cudaSuccess &&
                  cudaMalloc(&m->pf_tokens, T * 4) == cudaSuccess && cudaMalloc(&m->pf_tickets, (size_t)attn_batch * n_kv * 4) == cudaSuccess &&
                  cudaMemsetAsync(m->pf_tickets, 0, (size_t)attn_batch * n_kv * 4, ctx->stream) == cudaSuccess;
        if (!ok) {
            cudaGetLastError();
            llama_drop_prefill(m);
            return slai_set_error(ctx, SLAI_ERR_OOM, "prefill: cannot allocate buffers for %d tokens", t_pad);
        }
        m->pf_cap = t_pad;
        m->pf_attn_batch = attn_batch;
    }
    // attention partials of one batch of query tokens: sized by the last position of this prompt
    if (m->pf_attn_scratch_bytes < attn_bytes) {
        if (m->pf_attn_scratch) {
            cudaStreamSynchronize(ctx->stream);
            cudaFree(m->pf_attn_scratch);
            m->pf_attn_scratch = nullptr;
        }
        if (cudaMalloc(&m->pf_attn_scratch, attn_bytes) != cudaSuccess) {
            cudaGetLastError();
            m->pf_attn_scratch_bytes = 0;
            return slai_set_error(ctx, SLAI_ERR_OOM, "prefill: cannot allocate %zu bytes of attention scratch", attn_bytes);
        }
        m->pf_attn_scratch_bytes = attn_bytes;
    }
    return SLAI_OK;
}

static int llama_prefill_batched(slai_llama* m, const int32_t* h_tokens, int n, int pos0, float* h_last_logits) {
    slai_ctx* ctx = m->ctx;
    const slai_llama_config& c = m->cfg;
    const int NT = std::min(256, (n + 15) / 16 * 16);
    const int t_pad = (n + NT - 1) / NT * NT;
    const int AB = 64;  // query tokens per attention launch
    const int n_kv = attention_tickets(m->n_q_local, m->kv_mul);  // tickets per query token (virtual heads of the attention kernel)
    const size_t attn_per_token = attention_scratch_bytes(ctx, m->n_q_local, m->kv_mul, m->head_size, pos0 + n - 1);
    int rc = llama_prefill_reserve(m, t_pad, AB, attn_per_token * AB, n_kv);
    if (rc) return rc;
    const size_t esz = c.kv_dtype == SLAI_KV_F16 ? 2 : 4;
    const size_t kmax = (size_t)std::max(std::max(c.dim, m->hidden), m->q_dim);
    SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(m->pf_tokens, h_tokens, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
    SLAI_CHECK_CUDA(ctx, cudaMemsetAsync(m->pf_hi, 0, (size_t)m->pf_cap * kmax * 2, ctx->stream));  // rows beyond the prompt stay zero
    SLAI_CHECK_CUDA(ctx, cudaMemsetAsync(m->pf_lo, 0, (size_t)m->pf_cap * kmax * 2, ctx->stream));
    if ((rc = prefill_embed_launch(ctx, m->pf_x, c.dim, m->pf_tokens, n, m->embd_q ? nullptr : m->token_embd, m->embd_q))) return rc;
    const int qkv_ld = m->q_dim + 2 * m->kv_dim;
    auto gemm = [&](const slai_qmatrix* w, int rows, float* out, int ldo, int off, const float* resid, int ldr, const float* bias) {
        PrefillGemm G;
        // Fewer tokens per CTA tile while the grid would leave half of the SMs without a tile (4096-row matrices at 512 tokens:
        // 64 CTAs of 256 tokens become 128 CTAs of 128); every CTA dequantises its weight rows itself, so no further.
        int nt = NT;
        const int m_tiles = (rows + 127) / 128;
        while (nt > 64 && (nt / 2) % 16 == 0 && t_pad % (nt / 2) == 0 && m_tiles * (t_pad / nt) * 2 <= ctx->sm_count) nt /= 2;
        G.w = w; G.rows = rows; G.x_hi = m->pf_hi; G.x_lo = m->pf_lo; G.T = n; G.t_pad = t_pad; G.NT = nt;
        G.out = out; G.ldo = ldo; G.out_off = off; G.resid = resid; G.ldr = ldr; G.bias = bias;
        return prefill_gemm_launch(ctx, G);
    };
    // x += W * (the activations in pf_hi / pf_lo), W split by columns over the ranks of a sharded model
    auto row_parallel = [&](const slai_qmatrix* w) -> int {
        if (m->tp == 1) return gemm(w, c.dim, m->pf_x, c.dim, 0, m->pf_x, c.dim, nullptr);
        int r = gemm(w, c.dim, m->pf_part, c.dim, 0, nullptr, 0, nullptr);
        if (!r) r = tp_all_reduce_sum(ctx, m->pf_part, m->pf_part, (int64_t)n * c.dim);
        if (!r) r = slai_add_assign(ctx, m->pf_x, m->pf_part, (int64_t)n * c.dim);
        return r;
    };
    for (int l = 0; l < c.n_layers; l++) {
        const LlamaLayer& w = m->layers[l];
        void* kc = (char*)m->kcache + (size_t)l * m->kv_layer_elems * esz;
        void* vc = (char*)m->vcache + (size_t)l * m->kv_layer_elems * esz;
        // q, k, v                                                              transformer.rs:327-347
        if ((rc = prefill_split_launch(ctx, m->pf_x, c.dim, w.attn_norm, c.rms_norm_eps, n, c.dim, m->pf_hi, m->pf_lo))) return rc;
        if ((rc = gemm(w.wq, m->q_dim, m->pf_qkv, qkv_ld, 0, nullptr, 0, w.bq))) return rc;
        if ((rc = gemm(w.wk, m->kv_dim, m->pf_qkv, qkv_ld, m->q_dim, nullptr, 0, w.bk))) return rc;
        if ((rc = gemm(w.wv, m->kv_dim, m->pf_qkv, qkv_ld, m->q_dim + m->kv_dim, nullptr, 0, w.bv))) return rc;
        if ((rc = prefill_rope_kv_launch(ctx, m->pf_qkv, qkv_ld, m->q_dim, m->kv_dim, m->head_size, pos0, n, m->rope_theta, c.rope_variant != 0,
                                         m->pf_q, kc, vc, c.kv_dtype == SLAI_KV_F16, (long long)c.seq_len * m->head_size)))
            return rc;
        // attention                                                            transformer.rs:350
        const long long kv_head_stride = (long long)c.seq_len * m->head_size;
        const bool tiled = prefill_attention_supported(m->head_size, c.kv_dtype == SLAI_KV_F16, kc, vc, kv_head_stride) && m->q_dim % 4 == 0;
        if (tiled && (rc = prefill_attention_launch(ctx, m->pf_q, m->q_dim, kc, vc, c.kv_dtype == SLAI_KV_F16, kv_head_stride, m->head_size, m->n_q_local,
                                                    m->kv_mul, pos0, n, m->pf_xb, m->q_dim)))
            return rc;
        // (head sizes the tiled kernel does not take: the decode step's kernel, AB query tokens per launch)
        for (int t0 = 0; t0 < n && !tiled; t0 += AB) {
            const int nb = std::min(AB, n - t0);
            AttnLaunch A;
            A.q = m->pf_q + (size_t)t0 * m->q_dim; A.kcache = kc; A.vcache = vc; A.kv_dtype = c.kv_dtype;
            A.pos_stride = m->head_size; A.head_stride = (int64_t)c.seq_len * m->head_size;
            A.n_heads = m->n_q_local; A.kv_mul = m->kv_mul; A.head_size = m->head_size;
            A.d_pos = nullptr; A.max_pos = pos0 + n - 1; A.out = m->pf_xb + (size_t)t0 * m->q_dim; A.pdl = false;
            A.scratch = m->pf_attn_scratch; A.scratch_bytes = m->pf_attn_scratch_bytes;
            A.batch = nb; A.pos0 = pos0 + t0; A.q_batch_stride = m->q_dim; A.out_batch_stride = m->q_dim; A.batch_counters = m->pf_tickets;
            if ((rc = attention_launch(ctx, A))) return rc;
        }
        // x += Wo xb                                                           transformer.rs:352-355
        if ((rc = prefill_split_launch(ctx, m->pf_xb, m->q_dim, nullptr, 0.f, n, m->q_dim, m->pf_hi, m->pf_lo))) return rc;
        if ((rc = row_parallel(w.wo))) return rc;
        // FFN                                                                  transformer.rs:356-365
        if ((rc = prefill_split_launch(ctx, m->pf_x, c.dim, w.ffn_norm, c.rms_norm_eps, n, c.dim, m->pf_hi, m->pf_lo))) return rc;
        if ((rc = gemm(w.wgate, m->hidden, m->pf_g, m->hidden, 0, nullptr, 0, nullptr))) return rc;
        if ((rc = gemm(w.wup, m->hidden, m->pf_u, m->hidden, 0, nullptr, 0, nullptr))) return rc;
        if ((rc = prefill_silu_split_launch(ctx, m->pf_g, m->pf_u, n, m->hidden, m->pf_hi, m->pf_lo))) return rc;
        if ((rc = row_parallel(w.wdown))) return rc;
    }
    // the last token's state goes back to the decode step's vectors; final norm, logits and the greedy choice as there
    SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(m->x, m->pf_x + (size_t)(n - 1) * c.dim, (size_t)c.dim * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    const slai_qmatrix* wout = m->output ? m->output : (m->embd_q ? m->embd_q : &m->embd_as_matrix);
    if (wout->fmt == SLAI_FMT_F32) {
        if ((rc = slai_rms_norm(ctx, m->xb, m->x, m->out_norm, c.dim, c.rms_norm_eps))) return rc;
        GemvLaunch L;
        L.fmt = SLAI_FMT_F32; L.K = c.dim; L.nseg = 1; L.seg[0] = seg_of(wout, 0, c.vocab_size, nullptr, 0, 0);
        L.v = m->xb; L.out = m->logits; L.pdl = false;
        if ((rc = gemv_launch(ctx, L))) return rc;
    } else {
        GemvLaunch L;
        const int vrows = m->out_sharded ? c.vocab_size / m->tp : c.vocab_size;  // a sharded output matrix: this rank's rows, then gathered
        L.fmt = wout->fmt; L.K = c.dim; L.nseg = 1; L.seg[0] = seg_of(wout, 0, vrows, nullptr, 0, 0);
        L.v = m->x; L.out = m->out_sharded ? m->logits_part : m->logits; L.pro = PRO_RMS; L.norm_w = m->out_norm; L.eps = c.rms_norm_eps;
        L.epi = EPI_STORE; L.pdl = false;
        if ((rc = gemv_launch(ctx, L))) return rc;
        if (m->out_sharded && (rc = tp_all_gather(ctx, m->logits_part, m->logits, vrows))) return rc;
    }
    if ((rc = launch_argmax(ctx, m->logits, c.vocab_size, m->sc.d + 3, false))) return rc;
    if (h_last_logits) SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(h_last_logits, m->logits, (size_t)c.vocab_size * 4, cudaMemcpyDeviceToHost, ctx->stream));
    SLAI_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return slai_check_wait_flag(ctx);
}

SLAI_API int slai_llama_decode(slai_llama* m, int32_t token, int32_t pos, float* h_logits, int32_t* next_token) {
    if (!m) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    return decode_impl(m, llama_record, m->cfg.vocab_size, m->cfg.seq_len, token, pos, h_logits, next_token);
}
SLAI_API int slai_llama_generate_sampled(slai_llama* m, int32_t token, int32_t pos, int32_t n, float temperature, float topp, uint64_t seed,
                                         int32_t* h_tokens) {
    if (!m) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    slai_ctx* ctx = m->ctx;
    SLAI_REQUIRE(ctx, temperature >= 0.0f, SLAI_ERR_INVALID_ARG, "generate: negative temperature");
    if (!m->d_samp) {
        SLAI_CHECK_CUDA(ctx, cudaMalloc(&m->d_samp, sampler_params_bytes()));
        SLAI_CHECK_CUDA(ctx, cudaMalloc(&m->d_samp_scratch, sampler_scratch_bytes(m->cfg.vocab_size)));
    }
    int rc = sampler_set_params(ctx, m->d_samp, temperature, topp, seed);
    if (rc) return rc;
    return generate_impl(m, llama_record, m->cfg.vocab_size, m->cfg.seq_len, token, pos, n, h_tokens, G_SAMPLED);
}
SLAI_API int slai_llama_generate(slai_llama* m, int32_t token, int32_t pos, int32_t n, int32_t* h_tokens) {
    if (!m) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    return generate_impl(m, llama_record, m->cfg.vocab_size, m->cfg.seq_len, token, pos, n, h_tokens);
}
SLAI_API int slai_llama_prefill(slai_llama* m, const int32_t* h_tokens, int32_t n, int32_t pos0, float* h_last_logits) {
    if (!m) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    if (h_tokens && n >= 16 && pos0 >= 0 && pos0 + n <= m->cfg.seq_len && llama_prefill_eligible(m, n)) {
        for (int i = 0; i < n; i++)
            SLAI_REQUIRE(m->ctx, h_tokens[i] >= 0 && h_tokens[i] < m->cfg.vocab_size, SLAI_ERR_INVALID_ARG, "prefill: token %d out of range", h_tokens[i]);
        return llama_prefill_batched(m, h_tokens, n, pos0, h_last_logits);
    }
    return prefill_impl(m, llama_record, m->cfg.vocab_size, m->cfg.seq_len, h_tokens, n, pos0, h_last_logits);
}
// One decode step outside the graph and without programmatic dependent launch, with events around every GEMV and
// attention launch: device time per kernel class.  The step is a real one (the KV cache is written at `pos`).
SLAI_API int slai_llama_stats(slai_llama* m, int32_t token, int32_t pos, slai_llama_stats_t* out) {
    if (!m || !out) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    slai_ctx* ctx = m->ctx;
    SLAI_REQUIRE(ctx, token >= 0 && token < m->cfg.vocab_size, SLAI_ERR_INVALID_ARG, "stats: token %d out of range", token);
    SLAI_REQUIRE(ctx, pos >= 0 && pos < m->cfg.seq_len, SLAI_ERR_INVALID_ARG, "stats: pos %d out of range", pos);
    int rc = set_scalars(m, token, pos, 0);
    if (rc) return rc;
    SLAI_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const bool pdl = ctx->use_pdl;
    ctx->use_pdl = false;
    ctx->stats_on = true;
    rc = slai_stats_mark(ctx, STATS_OTHER);
    if (!rc) rc = llama_record(m, G_DECODE);
    if (!rc) rc = slai_stats_mark(ctx, STATS_OTHER);
    ctx->stats_on = false;
    ctx->use_pdl = pdl;
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    memset(out, 0, sizeof(*out));
    if (!rc && e == cudaSuccess) {
        for (size_t i = 1; i < ctx->stats_ev.size(); i++) {
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, ctx->stats_ev[i - 1], ctx->stats_ev[i]) != cudaSuccess) continue;
            const int cls = ctx->stats_cls[i];
            out->us[cls] += ms * 1000.f;
            out->us_total += ms * 1000.f;
            if (cls != STATS_OTHER) out->launches[cls]++;
        }
        out->launches[STATS_OTHER] = m->launches;
        for (int k = 1; k < STATS_CLASSES; k++) out->launches[STATS_OTHER] -= out->launches[k];
    }
    for (cudaEvent_t ev : ctx->stats_ev) cudaEventDestroy(ev);
    ctx->stats_ev.clear();
    ctx->stats_cls.clear();
    if (rc) return rc;
    if (e != cudaSuccess) return slai_set_error(ctx, SLAI_ERR_CUDA, "stats: %s", cudaGetErrorString(e));
    return slai_check_wait_flag(ctx);
}

SLAI_API int slai_llama_read_state(slai_llama* m, int which, float* h_out, int64_t n) {
    if (!m || !h_out) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    const float* src = nullptr;
    int64_t cap = 0;
    switch (which) {
        case 0: src = m->x; cap = m->cfg.dim; break;
        case 1: src = m->xb; cap = m->cfg.dim; break;
        case 2: src = m->q; cap = m->cfg.dim; break;
        case 3: src = m->hb; cap = m->cfg.hidden_dim; break;
        case 4: src = m->logits; cap = m->cfg.vocab_size; break;
        default: return slai_set_error(m->ctx, SLAI_ERR_INVALID_ARG, "read_state: unknown vector %d", which);
    }
    SLAI_REQUIRE(m->ctx, n > 0 && n <= cap, SLAI_ERR_SHAPE, "read_state: n=%lld exceeds %lld", (long long)n, (long long)cap);
    return slai_read_buffer(m->ctx, h_out, src, (size_t)n * 4);
}
SLAI_API int slai_llama_read_kv(slai_llama* m, int layer, int n_pos, float* h_keys, float* h_values) {
    if (!m || !h_keys || !h_values) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    slai_ctx* ctx = m->ctx;
    const slai_llama_config& c = m->cfg;
    SLAI_REQUIRE(ctx, layer >= 0 && layer < c.n_layers && n_pos > 0 && n_pos <= c.seq_len, SLAI_ERR_INVALID_ARG, "read_kv: layer %d / %d positions", layer, n_pos);
    const size_t esz = c.kv_dtype == SLAI_KV_F16 ? 2 : 4;
    const int n_kv = m->kv_dim / m->head_size, hs = m->head_size;
    std::vector<unsigned char> raw((size_t)n_pos * hs * esz);
    for (int which = 0; which < 2; which++) {
        const char* base = (const char*)(which ? m->vcache : m->kcache) + (size_t)layer * m->kv_layer_elems * esz;
        float* out = which ? h_values : h_keys;
        for (int h = 0; h < n_kv; h++) {  // cache: [kv_head][position][head_size]; out: [position][kv_head * head_size]
            SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(raw.data(), base + (size_t)h * c.seq_len * hs * esz, raw.size(), cudaMemcpyDeviceToHost, ctx->stream));
            SLAI_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            for (int p = 0; p < n_pos; p++)
                for (int d = 0; d < hs; d++)
                    out[(size_t)p * m->kv_dim + h * hs + d] = esz == 2 ? __half2float(reinterpret_cast<const __half*>(raw.data())[(size_t)p * hs + d])
                                                                       : reinterpret_cast<const float*>(raw.data())[(size_t)p * hs + d];
        }
    }
    return SLAI_OK;
}
SLAI_API int slai_llama_launches_per_token(const slai_llama* m) { return m ? m->launches : 0; }

// =================================================================================================
// GPT-2
// =================================================================================================
struct Gpt2Layer {
    const slai_qmatrix *w_qkv = nullptr, *w_proj = nullptr, *w_fc = nullptr, *w_fcproj = nullptr;
    float *ln1_g = nullptr, *ln1_b = nullptr, *b_qkv = nullptr, *b_proj = nullptr, *ln2_g = nullptr, *ln2_b = nullptr, *b_fc = nullptr,
          *b_fcproj = nullptr;
};
struct slai_gpt2 {
    slai_ctx* ctx = nullptr;
    slai_gpt2_config cfg;
    int head_size = 0;
    std::vector<Gpt2Layer> layers;
    const slai_qmatrix* wte = nullptr;  // token embedding and tied lm_head (models/gpt2/cpu.rs:197)
    float *wpe = nullptr, *lnf_g = nullptr, *lnf_b = nullptr;
    float *x = nullptr, *xb = nullptr, *q = nullptr, *ff = nullptr, *logits = nullptr;
    void *kcache = nullptr, *vcache = nullptr;
    size_t kv_layer_elems = 0;
    Scalars sc;
    int32_t* d_history = nullptr;
    int history_cap = 0;
    void* attn_scratch = nullptr;
    size_t attn_scratch_bytes = 0;
    GraphSet graphs;
    int launches = 0;
    // prompt processing as GEMMs (prefill.cu): buffers for `pf_cap` tokens, grown on demand
    int pf_cap = 0;
    float *pf_x = nullptr, *pf_qkv = nullptr, *pf_q = nullptr, *pf_xb = nullptr, *pf_ff = nullptr, *pf_theta0 = nullptr;
    __half *pf_hi = nullptr, *pf_lo = nullptr;
    int* pf_tokens = nullptr;
};

static void gpt2_drop_prefill(slai_gpt2* m) {
    if (m->pf_cap) cudaStreamSynchronize(m->ctx->stream);
    cudaFree(m->pf_x); cudaFree(m->pf_qkv); cudaFree(m->pf_q); cudaFree(m->pf_xb); cudaFree(m->pf_ff); cudaFree(m->pf_theta0);
    cudaFree(m->pf_hi); cudaFree(m->pf_lo); cudaFree(m->pf_tokens);
    m->pf_x = m->pf_qkv = m->pf_q = m->pf_xb = m->pf_ff = m->pf_theta0 = nullptr;
    m->pf_hi = m->pf_lo = nullptr;
    m->pf_tokens = nullptr;
    m->pf_cap = 0;
}

static int gpt2_record(slai_gpt2* m, int kind) {
    slai_ctx* ctx = m->ctx;
    const slai_gpt2_config& c = m->cfg;
    const bool pdl = ctx->use_pdl;
    const int E = c.n_embd;
    int n = 0, rc;
    int* d_token = m->sc.d;
    int* d_pos = m->sc.d + 1;
    SLAI_REQUIRE(ctx, m->wte && m->wpe && m->lnf_g && m->lnf_b, SLAI_ERR_INVALID_ARG, "gpt2: embeddings / final norm not set");
    // x = wte[:,tok] + wpe[:,pos]                                              gpt2/cpu.rs:227-228
    if ((rc = launch_embed_q8(ctx, m->x, m->wte, d_token, m->wpe, d_pos, false))) return rc;
    n++;
    const size_t esz = c.kv_dtype == SLAI_KV_F16 ? 2 : 4;
    for (int l = 0; l < c.n_layer; l++) {
        const Gpt2Layer& w = m->layers[l];
        SLAI_REQUIRE(ctx, w.w_qkv && w.w_proj && w.w_fc && w.w_fcproj && w.ln1_g && w.ln1_b && w.ln2_g && w.ln2_b && w.b_qkv &&
                              w.b_proj && w.b_fc && w.b_fcproj, SLAI_ERR_INVALID_ARG, "gpt2: layer %d has unset weights", l);
        void* kc = (char*)m->kcache + (size_t)l * m->kv_layer_elems * esz;
        void* vc = (char*)m->vcache + (size_t)l * m->kv_layer_elems * esz;
        {   // LayerNorm*g+b; qkv = W x + b; split into q / cache                gpt2/cpu.rs:235-270
            GemvLaunch L;
            L.fmt = w.w_qkv->fmt; L.K = E; L.nseg = 3;
            L.seg[0] = seg_of(w.w_qkv, 0, E, w.b_qkv, 0, 0);
            L.seg[1] = seg_of(w.w_qkv, E, E, w.b_qkv + E, 0, 1);
            L.seg[2] = seg_of(w.w_qkv, 2 * E, E, w.b_qkv + 2 * E, 0, 2);
            L.v = m->x; L.out = m->q; L.pro = PRO_LN; L.norm_w = w.ln1_g; L.norm_b = w.ln1_b; L.eps = c.layernorm_eps;
            L.epi = EPI_QKV; L.rope = 0; L.head_size = m->head_size; L.d_pos = d_pos; L.kcache = kc; L.vcache = vc;
            L.kv_dtype = c.kv_dtype; L.kv_pos_stride = m->head_size; L.kv_head_stride = (int64_t)c.n_seq * m->head_size;
            L.pdl = pdl;
            if ((rc = gemv_launch(ctx, L))) return rc;
            n++;
        }
        {   // attention with kv_mul = 1                                        gpt2/cpu.rs:272-290
            AttnLaunch A;
            A.q = m->q; A.kcache = kc; A.vcache = vc; A.kv_dtype = c.kv_dtype;
            A.pos_stride = m->head_size; A.head_stride = (int64_t)c.n_seq * m->head_size;
            A.n_heads = c.n_head; A.kv_mul = 1; A.head_size = m->head_size; A.d_pos = d_pos; A.max_pos = c.n_seq - 1;
            A.out = m->xb; A.pdl = pdl; A.pos_stable = true; A.scratch = m->attn_scratch; A.scratch_bytes = m->attn_scratch_bytes;
            if ((rc = attention_launch(ctx, A))) return rc;
            n++;
        }
        {   // x += W_proj xb + b                                               gpt2/cpu.rs:302-312
            GemvLaunch L;
            L.fmt = w.w_proj->fmt; L.K = E; L.nseg = 1; L.seg[0] = seg_of(w.w_proj, 0, E, w.b_proj, 0, 0);
            L.v = m->xb; L.out = m->x; L.resid = m->x; L.epi = EPI_RESID; L.pdl = pdl;
            if ((rc = gemv_launch(ctx, L))) return rc;
            n++;
        }
        {   // ff = gelu(W_fc (LayerNorm(x)*g+b) + b)                            gpt2/cpu.rs:318-343
            GemvLaunch L;
            L.fmt = w.w_fc->fmt; L.K = E; L.nseg = 1; L.seg[0] = seg_of(w.w_fc, 0, c.ff_len, w.b_fc, 0, 0);
            L.v = m->x; L.out = m->ff; L.pro = PRO_LN; L.norm_w = w.ln2_g; L.norm_b = w.ln2_b; L.eps = c.layernorm_eps;
            L.epi = EPI_GELU; L.pdl = pdl;
            if ((rc = gemv_launch(ctx, L))) return rc;
            n++;
        }
        {   // x += W_proj2 ff + b                                              gpt2/cpu.rs:353-360
            GemvLaunch L;
            L.fmt = w.w_fcproj->fmt; L.K = c.ff_len; L.nseg = 1; L.seg[0] = seg_of(w.w_fcproj, 0, E, w.b_fcproj, 0, 0);
            L.v = m->ff; L.out = m->x; L.resid = m->x; L.epi = EPI_RESID; L.pdl = pdl;
            if ((rc = gemv_launch(ctx, L))) return rc;
            n++;
        }
    }
    {   // logits = wte (LayerNorm(x)*g+b)                                      gpt2/cpu.rs:366-379
        GemvLaunch L;
        L.fmt = m->wte->fmt; L.K = E; L.nseg = 1; L.seg[0] = seg_of(m->wte, 0, c.n_vocab, nullptr, 0, 0);
        L.v = m->x; L.out = m->logits; L.pro = PRO_LN; L.norm_w = m->lnf_g; L.norm_b = m->lnf_b; L.eps = c.layernorm_eps;
        L.epi = EPI_STORE; L.pdl = pdl;
        if ((rc = gemv_launch(ctx, L))) return rc;
        n++;
    }
    if ((rc = launch_argmax(ctx, m->logits, c.n_vocab, m->sc.d + 3, pdl))) return rc;
    n++;
    if (kind == G_GENERATE) {
        if ((rc = launch_advance(ctx, d_token, d_pos, m->sc.d + 3, m->d_history, c.n_vocab, pdl))) return rc;
        n++;
    } else if (kind == G_FORCED) {
        if ((rc = launch_advance(ctx, d_token, d_pos, nullptr, m->d_history, c.n_vocab, pdl))) return rc;
        n++;
    }
    m->launches = n;
    return SLAI_OK;
}

SLAI_API int slai_gpt2_create(slai_ctx* ctx, const slai_gpt2_config* cfg, slai_gpt2** out) {
    if (!ctx || !cfg || !out) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    *out = nullptr;
    const slai_gpt2_config& c = *cfg;
    SLAI_REQUIRE(ctx, c.n_vocab > 0 && c.n_seq > 0 && c.n_embd > 0 && c.n_head > 0 && c.n_layer > 0 && c.ff_len > 0, SLAI_ERR_INVALID_ARG,
                 "gpt2: non-positive dimension");
    SLAI_REQUIRE(ctx, c.n_embd % c.n_head == 0 && (c.n_embd / c.n_head) % 2 == 0, SLAI_ERR_SHAPE, "gpt2: bad head size");
    SLAI_REQUIRE(ctx, c.kv_dtype == SLAI_KV_F16 || c.kv_dtype == SLAI_KV_F32, SLAI_ERR_INVALID_ARG, "gpt2: unknown kv_dtype");
    slai_gpt2* m = new slai_gpt2();
    m->ctx = ctx;
    m->cfg = c;
    m->head_size = c.n_embd / c.n_head;
    m->layers.resize(c.n_layer);
    const size_t esz = c.kv_dtype == SLAI_KV_F16 ? 2 : 4;
    m->kv_layer_elems = (size_t)c.n_seq * c.n_embd;
    const char* ng = getenv("SLAI_NO_GRAPH");
    m->graphs.use_graph = !(ng && ng[0] == '1');
    m->history_cap = c.n_seq + 8;
    m->attn_scratch_bytes = attention_scratch_bytes(ctx, c.n_head, 1, m->head_size, c.n_seq - 1);
    bool ok = cudaMalloc(&m->x, (size_t)c.n_embd * 4) == cudaSuccess && cudaMalloc(&m->xb, (size_t)c.n_embd * 4) == cudaSuccess &&
              cudaMalloc(&m->q, (size_t)c.n_embd * 4) == cudaSuccess && cudaMalloc(&m->ff, (size_t)c.ff_len * 4) == cudaSuccess &&
              cudaMalloc(&m->logits, (size_t)c.n_vocab * 4) == cudaSuccess &&
              cudaMalloc(&m->kcache, m->kv_layer_elems * c.n_layer * esz) == cudaSuccess &&
              cudaMalloc(&m->vcache, m->kv_layer_elems * c.n_layer * esz) == cudaSuccess && cudaMalloc(&m->sc.d, 64) == cudaSuccess &&
              cudaMalloc(&m->d_history, (size_t)m->history_cap * 4) == cudaSuccess &&
              cudaMalloc(&m->attn_scratch, m->attn_scratch_bytes) == cudaSuccess;
    if (ok)
        ok = cudaMemsetAsync(m->kcache, 0, m->kv_layer_elems * c.n_layer * esz, ctx->stream) == cudaSuccess &&
             cudaMemsetAsync(m->vcache, 0, m->kv_layer_elems * c.n_layer * esz, ctx->stream) == cudaSuccess &&
             cudaMemsetAsync(m->sc.d, 0, 64, ctx->stream) == cudaSuccess &&
             cudaMemsetAsync(m->d_history, 0, (size_t)m->history_cap * 4, ctx->stream) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        slai_gpt2_destroy(m);
        return slai_set_error(ctx, SLAI_ERR_OOM, "gpt2: cannot allocate the model state");
    }
    *out = m;
    return SLAI_OK;
}

SLAI_API int slai_gpt2_destroy(slai_gpt2* m) {
    if (!m) return SLAI_OK;
    SLAI_ENTER(m->ctx);
    cudaStreamSynchronize(m->ctx->stream);
    destroy_graphs(m->graphs);
    for (auto& l : m->layers) {
        cudaFree(l.ln1_g); cudaFree(l.ln1_b); cudaFree(l.b_qkv); cudaFree(l.b_proj); cudaFree(l.ln2_g); cudaFree(l.ln2_b);
        cudaFree(l.b_fc); cudaFree(l.b_fcproj);
    }
    cudaFree(m->wpe); cudaFree(m->lnf_g); cudaFree(m->lnf_b);
    cudaFree(m->x); cudaFree(m->xb); cudaFree(m->q); cudaFree(m->ff); cudaFree(m->logits);
    cudaFree(m->kcache); cudaFree(m->vcache); cudaFree(m->sc.d); cudaFree(m->d_history); cudaFree(m->attn_scratch);
    gpt2_drop_prefill(m);
    delete m;
    return SLAI_OK;
}

SLAI_API int slai_gpt2_set_matrix(slai_gpt2* m, int id, int layer, const slai_qmatrix* w) {
    if (!m || !w) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    slai_ctx* ctx = m->ctx;
    const slai_gpt2_config& c = m->cfg;
    destroy_graphs(m->graphs);
    auto shape_is = [&](int64_t r, int64_t k) { return w->nrows == r && w->ncols == k; };
    if (id == SLAI_G_WTE) {
        SLAI_REQUIRE(ctx, shape_is(c.n_vocab, c.n_embd), SLAI_ERR_SHAPE, "gpt2: wte must be n_vocab x n_embd");
        m->wte = w;
        return SLAI_OK;
    }
    SLAI_REQUIRE(ctx, layer >= 0 && layer < c.n_layer, SLAI_ERR_INVALID_ARG, "gpt2: layer %d out of range", layer);
    Gpt2Layer& l = m->layers[layer];
    switch (id) {
        case SLAI_G_W_QKV:
            SLAI_REQUIRE(ctx, shape_is(3 * c.n_embd, c.n_embd), SLAI_ERR_SHAPE, "gpt2: attn_qkv must be 3E x E");
            SLAI_REQUIRE(ctx, c.n_embd % 16 == 0, SLAI_ERR_SHAPE, "gpt2: n_embd must be a multiple of 16 (q/k/v rows start on tile boundaries)");
            l.w_qkv = w;
            break;
        case SLAI_G_W_PROJ: SLAI_REQUIRE(ctx, shape_is(c.n_embd, c.n_embd), SLAI_ERR_SHAPE, "gpt2: attn_output must be E x E"); l.w_proj = w; break;
        case SLAI_G_W_FC: SLAI_REQUIRE(ctx, shape_is(c.ff_len, c.n_embd), SLAI_ERR_SHAPE, "gpt2: ffn_up must be ff x E"); l.w_fc = w; break;
        case SLAI_G_W_FCPROJ: SLAI_REQUIRE(ctx, shape_is(c.n_embd, c.ff_len), SLAI_ERR_SHAPE, "gpt2: ffn_down must be E x ff"); l.w_fcproj = w; break;
        default: return slai_set_error(ctx, SLAI_ERR_INVALID_ARG, "gpt2: weight id %d is not a matrix", id);
    }
    return SLAI_OK;
}

SLAI_API int slai_gpt2_set_f32(slai_gpt2* m, int id, int layer, const float* h_data, int64_t n) {
    if (!m || !h_data) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    slai_ctx* ctx = m->ctx;
    const slai_gpt2_config& c = m->cfg;
    destroy_graphs(m->graphs);
    float** dst = nullptr;
    int64_t want = c.n_embd;
    if (id == SLAI_G_WPE) { dst = &m->wpe; want = (int64_t)c.n_seq * c.n_embd; }
    else if (id == SLAI_G_LNF_G) dst = &m->lnf_g;
    else if (id == SLAI_G_LNF_B) dst = &m->lnf_b;
    else {
        SLAI_REQUIRE(ctx, layer >= 0 && layer < c.n_layer, SLAI_ERR_INVALID_ARG, "gpt2: layer %d out of range", layer);
        Gpt2Layer& l = m->layers[layer];
        switch (id) {
            case SLAI_G_LN1_G: dst = &l.ln1_g; break;
            case SLAI_G_LN1_B: dst = &l.ln1_b; break;
            case SLAI_G_B_QKV: dst = &l.b_qkv; want = 3 * (int64_t)c.n_embd; break;
            case SLAI_G_B_PROJ: dst = &l.b_proj; break;
            case SLAI_G_LN2_G: dst = &l.ln2_g; break;
            case SLAI_G_LN2_B: dst = &l.ln2_b; break;
            case SLAI_G_B_FC: dst = &l.b_fc; want = c.ff_len; break;
            case SLAI_G_B_FCPROJ: dst = &l.b_fcproj; break;
            default: return slai_set_error(ctx, SLAI_ERR_INVALID_ARG, "gpt2: weight id %d is not an f32 vector", id);
        }
    }
    SLAI_REQUIRE(ctx, n == want, SLAI_ERR_SHAPE, "gpt2: weight %d needs %lld floats, got %lld", id, (long long)want, (long long)n);
    return copy_f32(ctx, dst, h_data, n, false);
}

SLAI_API int slai_gpt2_decode(slai_gpt2* m, int32_t token, int32_t pos, float* h_logits, int32_t* next_token) {
    if (!m) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    return decode_impl(m, gpt2_record, m->cfg.n_vocab, m->cfg.n_seq, token, pos, h_logits, next_token);
}
SLAI_API int slai_gpt2_generate(slai_gpt2* m, int32_t token, int32_t pos, int32_t n, int32_t* h_tokens) {
    if (!m) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    return generate_impl(m, gpt2_record, m->cfg.n_vocab, m->cfg.n_seq, token, pos, n, h_tokens);
}
// ---- prompt processing as GEMMs ---------------------------------------------------------------------------------------
// The T prompt tokens go through every layer together, as for Llama (prefill.cu): per layer LayerNorm (gamma, beta) +
// fp16-pair split, the fused q/k/v GEMM with its bias, cache write (the rotation kernel with a table of zero angles: the
// identity), tiled causal attention, projection GEMM with bias and residual, LayerNorm + split, feed-forward GEMM with
// bias, GELU + split, second feed-forward GEMM with bias and residual (models/gpt2/cpu.rs:225-383 for one token).
static bool gpt2_prefill_eligible(const slai_gpt2* m, int n) {
    const char* e = getenv("SLAI_PREFILL_SEQUENTIAL");
    if (e && e[0] == '1') return false;
    if (n < 16 || !m->wte || !m->wpe || !m->lnf_g || !m->lnf_b) return false;
    const size_t esz = m->cfg.kv_dtype == SLAI_KV_F16 ? 2 : 4;
    (void)esz;
    if (!prefill_attention_supported(m->head_size, m->cfg.kv_dtype == SLAI_KV_F16, m->kcache, m->vcache, (long long)m->cfg.n_seq * m->head_size) ||
        m->cfg.n_embd % 4 != 0)
        return false;
    for (auto& w : m->layers) {
        const slai_qmatrix* ms[4] = {w.w_qkv, w.w_proj, w.w_fc, w.w_fcproj};
        for (auto* q : ms)
            if (!q || q->fmt == SLAI_FMT_F32 || q->ncols % 64 != 0) return false;
        if (!w.ln1_g || !w.ln1_b || !w.ln2_g || !w.ln2_b || !w.b_qkv || !w.b_proj || !w.b_fc || !w.b_fcproj) return false;
    }
    return true;
}

static int gpt2_prefill_batched(slai_gpt2* m, const int32_t* h_tokens, int n, int pos0, float* h_last_logits) {
    slai_ctx* ctx = m->ctx;
    const slai_gpt2_config& c = m->cfg;
    const int E = c.n_embd, F = c.ff_len;
    const int NT = std::min(256, (n + 15) / 16 * 16);
    const int t_pad = (n + NT - 1) / NT * NT;
    const size_t kmax = (size_t)std::max(E, F);
    if (t_pad > m->pf_cap) gpt2_drop_prefill(m);
    if (!m->pf_cap) {
        const size_t T = (size_t)t_pad;
        bool ok = cudaMalloc(&m->pf_x, T * E * 4) == cudaSuccess && cudaMalloc(&m->pf_qkv, T * 3 * E * 4) == cudaSuccess &&
                  cudaMalloc(&m->pf_q, T * E * 4) == cudaSuccess && cudaMalloc(&m->pf_xb, T * E * 4) == cudaSuccess &&
                  cudaMalloc(&m->pf_ff, T * F * 4) == cudaSuccess && cudaMalloc(&m->pf_hi, T * kmax * 2) == cudaSuccess &&
                  cudaMalloc(&m->pf_lo, T * kmax * 2) == cudaSuccess && cudaMalloc(&m->pf_tokens, T * 4) == cudaSuccess &&
                  cudaMalloc(&m->pf_theta0, (size_t)m->head_size * 4) == cudaSuccess &&
                  cudaMemsetAsync(m->pf_theta0, 0, (size_t)m->head_size * 4, ctx->stream) == cudaSuccess;
        if (!ok) {
            cudaGetLastError();
            gpt2_drop_prefill(m);
            return slai_set_error(ctx, SLAI_ERR_OOM, "prefill: cannot allocate buffers for %d tokens", t_pad);
        }
        m->pf_cap = t_pad;
    }
    int rc;
    const size_t esz = c.kv_dtype == SLAI_KV_F16 ? 2 : 4;
    SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(m->pf_tokens, h_tokens, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
    SLAI_CHECK_CUDA(ctx, cudaMemsetAsync(m->pf_hi, 0, (size_t)m->pf_cap * kmax * 2, ctx->stream));  // rows beyond the prompt stay zero
    SLAI_CHECK_CUDA(ctx, cudaMemsetAsync(m->pf_lo, 0, (size_t)m->pf_cap * kmax * 2, ctx->stream));
    // x = wte[:,tok] + wpe[:,pos]                                              gpt2/cpu.rs:227-228
    if ((rc = prefill_embed_launch(ctx, m->pf_x, E, m->pf_tokens, n, nullptr, m->wte))) return rc;
    if ((rc = prefill_add_rows_launch(ctx, m->pf_x, E, m->wpe, pos0, n))) return rc;
    auto gemm = [&](const slai_qmatrix* w, int rows, float* out, int ldo, const float* resid, int ldr, const float* bias) {
        PrefillGemm G;
        int nt = NT;
        const int m_tiles = (rows + 127) / 128;
        while (nt > 64 && (nt / 2) % 16 == 0 && t_pad % (nt / 2) == 0 && m_tiles * (t_pad / nt) * 2 <= ctx->sm_count) nt /= 2;
        G.w = w; G.rows = rows; G.x_hi = m->pf_hi; G.x_lo = m->pf_lo; G.T = n; G.t_pad = t_pad; G.NT = nt;
        G.out = out; G.ldo = ldo; G.out_off = 0; G.resid = resid; G.ldr = ldr; G.bias = bias;
        return prefill_gemm_launch(ctx, G);
    };
    const long long kv_head_stride = (long long)c.n_seq * m->head_size;
    for (int l = 0; l < c.n_layer; l++) {
        const Gpt2Layer& w = m->layers[l];
        void* kc = (char*)m->kcache + (size_t)l * m->kv_layer_elems * esz;
        void* vc = (char*)m->vcache + (size_t)l * m->kv_layer_elems * esz;
        if ((rc = prefill_split_ln_launch(ctx, m->pf_x, E, w.ln1_g, w.ln1_b, c.layernorm_eps, n, E, m->pf_hi, m->pf_lo))) return rc;
        if ((rc = gemm(w.w_qkv, 3 * E, m->pf_qkv, 3 * E, nullptr, 0, w.b_qkv))) return rc;
        if ((rc = prefill_rope_kv_launch(ctx, m->pf_qkv, 3 * E, E, E, m->head_size, pos0, n, m->pf_theta0, 0, m->pf_q, kc, vc,
                                         c.kv_dtype == SLAI_KV_F16, kv_head_stride)))
            return rc;
        if ((rc = prefill_attention_launch(ctx, m->pf_q, E, kc, vc, c.kv_dtype == SLAI_KV_F16, kv_head_stride, m->head_size, c.n_head, 1, pos0, n,
                                           m->pf_xb, E)))
            return rc;
        if ((rc = prefill_split_launch(ctx, m->pf_xb, E, nullptr, 0.f, n, E, m->pf_hi, m->pf_lo))) return rc;
        if ((rc = gemm(w.w_proj, E, m->pf_x, E, m->pf_x, E, w.b_proj))) return rc;
        if ((rc = prefill_split_ln_launch(ctx, m->pf_x, E, w.ln2_g, w.ln2_b, c.layernorm_eps, n, E, m->pf_hi, m->pf_lo))) return rc;
        if ((rc = gemm(w.w_fc, F, m->pf_ff, F, nullptr, 0, w.b_fc))) return rc;
        if ((rc = prefill_gelu_split_launch(ctx, m->pf_ff, n, F, m->pf_hi, m->pf_lo))) return rc;
        if ((rc = gemm(w.w_fcproj, E, m->pf_x, E, m->pf_x, E, w.b_fcproj))) return rc;
    }
    // the last token's state goes back to the decode step's vector; final norm, logits and the greedy choice as there
    SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(m->x, m->pf_x + (size_t)(n - 1) * E, (size_t)E * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    {
        GemvLaunch L;
        L.fmt = m->wte->fmt; L.K = E; L.nseg = 1; L.seg[0] = seg_of(m->wte, 0, c.n_vocab, nullptr, 0, 0);
        L.v = m->x; L.out = m->logits; L.pro = PRO_LN; L.norm_w = m->lnf_g; L.norm_b = m->lnf_b; L.eps = c.layernorm_eps;
        L.epi = EPI_STORE; L.pdl = false;
        if ((rc = gemv_launch(ctx, L))) return rc;
    }
    if ((rc = launch_argmax(ctx, m->logits, c.n_vocab, m->sc.d + 3, false))) return rc;
    if (h_last_logits) SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(h_last_logits, m->logits, (size_t)c.n_vocab * 4, cudaMemcpyDeviceToHost, ctx->stream));
    SLAI_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return slai_check_wait_flag(ctx);
}

SLAI_API int slai_gpt2_prefill(slai_gpt2* m, const int32_t* h_tokens, int32_t n, int32_t pos0, float* h_last_logits) {
    if (!m) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(m->ctx);
    if (h_tokens && n >= 16 && pos0 >= 0 && pos0 + n <= m->cfg.n_seq && gpt2_prefill_eligible(m, n)) {
        for (int i = 0; i < n; i++)
            SLAI_REQUIRE(m->ctx, h_tokens[i] >= 0 && h_tokens[i] < m->cfg.n_vocab, SLAI_ERR_INVALID_ARG, "prefill: token %d out of range", h_tokens[i]);
        return gpt2_prefill_batched(m, h_tokens, n, pos0, h_last_logits);
    }
    return prefill_impl(m, gpt2_record, m->cfg.n_vocab, m->cfg.n_seq, h_tokens, n, pos0, h_last_logits);
}
