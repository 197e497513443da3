// Host side of the fused decode step: carves the scratch arena, chains the
// kernels of 24 layers + lm_head with programmatic dependent launch, and can
// capture several consecutive steps into one CUDA graph.
//
// One step replaces Engine.step + QUICForCausalLM.forward(seq_len == 1) of the
// reference (src/engine.py:78-107, src/model.py:272-303).  Token ids, positions
// and the row -> slot map live in device memory, so a captured graph is valid
// for any position and consecutive steps need no host round trip.
#include <cstdio>
#include <new>

#include "decode_kernels.cuh"

namespace quic {
void attn_carve_scratch(void* scratch, int b, int splits, AttnArgs* a);

namespace {

inline int64_t align256(int64_t v) { return (v + 255) / 256 * 256; }

struct Arena {
  int64_t lm_counter, attn, xres, qbuf, attn_out, act, partial, best_val, best_idx, total;
  // batched step (batch > kMaxM) only
  int64_t xn, qkv, gu, act16, tcws;
};

int64_t tc_workspace_bytes(int batch) {
  int64_t w = w4a16_gemm_tc_workspace(batch, kQkvN, kHidden);
  const int64_t o = w4a16_gemm_tc_workspace(batch, kHidden, kHidden);
  const int64_t g = w4a16_gemm_tc_workspace(batch, 2 * kInter, kHidden);
  const int64_t d = w4a16_gemm_tc_workspace(batch, kHidden, kInter);
  w = w > o ? w : o;
  w = w > g ? w : g;
  w = w > d ? w : d;
  // the dense fp16 GEMM's split-K planes (same arena slot)
  const int shapes[4][2] = {{kQkvN, kHidden}, {kHidden, kHidden}, {2 * kInter, kHidden}, {kHidden, kInter}};
  for (const auto& s : shapes) {
    const int64_t f = gemm_f16_tc_workspace(batch, s[0], s[1]);
    w = w > f ? w : f;
  }
  return w;
}

// The regions that must start zeroed (arrival counters) come first.
Arena carve(int batch, int vocab, int splits) {
  Arena a;
  int64_t off = 0;
  a.lm_counter = off;  // arrival counter, then the lm_head's per-row maxima (up to 128 rows)
  off += 256 + 128 * 8;
  a.attn = off;
  off += align256(quic_attn_scratch_bytes(batch, splits));
  a.xres = off;
  off += align256((int64_t)2 * batch * kHidden * 2);
  a.qbuf = off;
  off += align256((int64_t)batch * kHidden * 2);
  a.attn_out = off;
  off += align256((int64_t)batch * kHidden * 2);
  a.act = off;
  off += align256((int64_t)4 * batch * kInter * 4);
  a.partial = off;
  off += align256((int64_t)kDownSplits * batch * kHidden * 4);
  int grid = lm_head_grid(vocab);
  if (lm_head_tc_supported(batch, vocab) && lm_head_tc_tiles(vocab) > grid) grid = lm_head_tc_tiles(vocab);
  a.best_val = off;
  off += align256((int64_t)batch * grid * 4);
  a.best_idx = off;
  off += align256((int64_t)batch * grid * 4);
  a.xn = a.qkv = a.gu = a.act16 = a.tcws = off;
  if (batch >= 2) {  // the tensor-core step may be selected from batch 2 upwards
    a.xn = off;
    off += align256((int64_t)batch * kHidden * 2);
    a.qkv = off;
    off += align256((int64_t)batch * kQkvN * 2);
    a.gu = off;
    off += align256((int64_t)batch * 2 * kInter * 2);
    a.act16 = off;
    off += align256((int64_t)batch * kInter * 2);
    a.tcws = off;
    off += align256(16384 + tc_workspace_bytes(batch));
  }
  a.total = off;
  return a;
}

int pick_splits(const quic_decode_t* d) {
  if (d->attn_splits > 0) return d->attn_splits;
  int ctx = d->ctx_hint > 0 ? d->ctx_hint : d->s_max;
  if (ctx > d->s_max) ctx = d->s_max;
  return quic_decode_pick_splits(d->batch, ctx);
}

int check(const quic_model_t* m, const quic_decode_t* d) {
  QUIC_REQUIRE(m && d, QUIC_E_ARG, "decode_step: null argument");
  QUIC_REQUIRE(m->n_layers >= 1 && m->layers, QUIC_E_ARG, "decode_step: no layers");
  QUIC_REQUIRE(m->vocab >= 2 && m->vocab % 2 == 0, QUIC_E_SHAPE, "decode_step: vocab must be even");
  QUIC_REQUIRE(m->embed && m->final_norm && m->rope_cos && m->rope_sin && m->max_pos >= 1,
               QUIC_E_ARG, "decode_step: missing model tensor");
  QUIC_REQUIRE(d->kv && d->tok && d->pos && d->rows && d->scratch, QUIC_E_ARG,
               "decode_step: missing state tensor");
  QUIC_REQUIRE(d->batch >= 1 && d->batch <= 8 * 65535 && d->n_slots >= 1 && d->s_max >= 1,
               QUIC_E_SHAPE, "decode_step: bad batch / cache geometry");
  QUIC_REQUIRE(d->out_tokens == nullptr || (d->ring >= 1 && d->step_counter != nullptr),
               QUIC_E_ARG, "decode_step: out_tokens needs ring >= 1 and a step counter");
  for (int l = 0; l < m->n_layers; ++l) {
    const quic_layer_t& L = m->layers[l];
    QUIC_REQUIRE(L.qkv.n == kQkvN && L.qkv.k == kHidden && L.o.n == kHidden && L.o.k == kHidden &&
                     L.gate_up.n == 2 * kInter && L.gate_up.k == kHidden && L.down.n == kHidden &&
                     L.down.k == kInter,
                 QUIC_E_SHAPE, "decode_step: layer shapes are not Qwen2.5-0.5B's");
    const bool packed = L.qkv.qw && L.o.qw && L.gate_up.qw && L.down.qw;
    const bool dense = L.qkv.w16 && L.o.w16 && L.gate_up.w16 && L.down.w16;
    QUIC_REQUIRE((packed || dense) && L.ln1 && L.ln2, QUIC_E_ARG, "decode_step: missing layer tensor");
    QUIC_REQUIRE(dense == (m->layers[0].qkv.w16 != nullptr), QUIC_E_ARG,
                 "decode_step: packed and dense layers cannot be mixed");
  }
  return QUIC_OK;
}


int enqueue_step_batched(const quic_model_t* m, const quic_decode_t* d, cudaStream_t st, bool chain_head);
int enqueue_step_rows16(const quic_model_t* m, const quic_decode_t* d, cudaStream_t st, bool chain_head);

// Smallest batch that takes the tensor-core (tcgen05) step (quic_set_tensor_min_batch): 2..17,
// and smallest batch that takes the mma.sync chain (quic_set_mma_chain_min_batch): 2..17.
// Below both, the rows run the GEMV chain (FMA; its cost grows with every row, measured 352,
// 491 and 683 us per step at 1, 2 and 3 rows against 565 and 580 us of the mma.sync chain).
// (the tensor-core step, 731..759 us at 6..16 rows of 512 tokens, meets the mma.sync chain, 642..776, at 16 rows)
int g_tensor_min_batch = kMmaChainMaxRows;
int g_mma_chain_min_batch = 3;

int enqueue_step_f16(const quic_model_t* m, const quic_decode_t* d, cudaStream_t st, bool chain_head);
int enqueue_step_batched_f16(const quic_model_t* m, const quic_decode_t* d, cudaStream_t st, bool chain_head);

int enqueue_step(const quic_model_t* m, const quic_decode_t* d, cudaStream_t st, bool chain_head) {
  const int B = d->batch;
  if (m->layers[0].qkv.w16 != nullptr)  // dense fp16 weights
    return B <= kF16ChainMaxRows ? enqueue_step_f16(m, d, st, chain_head) : enqueue_step_batched_f16(m, d, st, chain_head);
  if (B >= g_tensor_min_batch) return enqueue_step_batched(m, d, st, chain_head);
  if (B >= g_mma_chain_min_batch) return enqueue_step_rows16(m, d, st, chain_head);
  const int splits = pick_splits(d);
  const Arena ar = carve(B, m->vocab, splits);
  char* base = static_cast<char*>(d->scratch);
  half* xres[2] = {reinterpret_cast<half*>(base + ar.xres),
                   reinterpret_cast<half*>(base + ar.xres) + (size_t)B * kHidden};
  half* qbuf = reinterpret_cast<half*>(base + ar.qbuf);
  half* attn_out = reinterpret_cast<half*>(base + ar.attn_out);
  float* gu_part = reinterpret_cast<float*>(base + ar.act);
  float* partial = reinterpret_cast<float*>(base + ar.partial);

  const size_t slot_stride = (size_t)kKvHeads * d->s_max * kHeadDim;  // one slot, K or V
  const size_t kv_plane = (size_t)d->n_slots * slot_stride;           // K (or V) of a layer
  int ctx = d->ctx_hint > 0 ? d->ctx_hint : d->s_max;
  if (ctx > d->s_max) ctx = d->s_max;

  RowState rs;
  rs.rows = d->rows;
  rs.tok = d->tok;
  rs.pos = d->pos;
  rs.batch = B;

  for (int l = 0; l < m->n_layers; ++l) {
    const quic_layer_t& L = m->layers[l];
    half* kc = static_cast<half*>(d->kv) + (size_t)(2 * l) * kv_plane;
    half* vc = kc + kv_plane;

    QkvArgs qa = {};
    qa.w = L.qkv;
    qa.ln = (const half*)L.ln1;
    qa.embed = (const half*)m->embed;
    qa.xres_in = xres[1];
    qa.xres_out = xres[0];
    qa.partial = partial;
    qa.rs = rs;
    qa.eps = m->eps;
    qa.first_layer = (l == 0);
    qa.vocab = m->vocab;
    qa.cos_t = (const half*)m->rope_cos;
    qa.sin_t = (const half*)m->rope_sin;
    qa.max_pos = m->max_pos;
    qa.qbuf = qbuf;
    qa.kcache = kc;
    qa.vcache = vc;
    qa.s_max = d->s_max;
    // The first kernel of a sequence starts only after everything enqueued before it has
    // completed (no programmatic overlap), so later kernels of the chain may read the cache
    // before their own dependency wait.
    QUIC_CUDA(launch_qkv(qa, st, !(chain_head && l == 0)));

    AttnArgs aa = {};
    aa.q = qbuf;
    aa.k = kc;
    aa.v = vc;
    aa.stride_b = (int64_t)slot_stride;
    aa.stride_h = (int64_t)d->s_max * kHeadDim;
    aa.rows = d->rows;
    aa.pos = d->pos;
    aa.s_cap = ctx;
    aa.splits = splits;
    aa.chunk = (ctx + splits - 1) / splits;
    aa.scale = 0.125f;  // 64^-0.5, src/model.py:129
    aa.out = attn_out;
    // 64-token single-warp CTAs (latency variant) up to 2048 tokens, merged by the o_proj kernel
    aa.small = (splits <= kWarpMaxSplits && (int64_t)splits * 64 >= ctx) ? 1 : 0;
    aa.use_mma = 1;  // beyond 2048 tokens: the mma.sync throughput kernel
    const bool consumer_merge = splits > 1 && splits <= kMaxConsumerSplitsTotal;
    aa.consumer_merge = consumer_merge ? 1 : 0;
    aa.epoch = d->step_counter;
    aa.prefetch = (aa.small && d->step_counter != nullptr) ? 1 : 0;
    // Up to 4096 tokens: CTAs of 512 tokens (eight warps merged in shared memory, every cache tile
    // requested before the wait), beyond 512 tokens a cluster merged in distributed shared memory;
    // the o_proj kernel reads the finished heads.  Measured 318 / 347 / 352 us per token at 200 /
    // 512..576 / 1500 tokens against 347 / 350 / 375 with one-warp CTAs merged by the o_proj kernel.
    const int cta_splits = attn_cta_splits(ctx);
    const bool cta_attn = cta_splits <= kAttnCtaMaxSplits;
    if (cta_attn) {
      aa.splits = cta_splits;
      aa.chunk = 512;
      aa.small = 0;
      aa.consumer_merge = 0;
      aa.prefetch = d->step_counter != nullptr ? 1 : 0;
      QUIC_CUDA(launch_attn_cta(aa, B, st, true));
    } else {
      if (splits > 1) attn_carve_scratch(base + ar.attn, B, splits, &aa);
      QUIC_CUDA(launch_attn(aa, B, st, true));
    }

    OProjArgs oa = {};
    oa.w = L.o;
    oa.attn = attn_out;
    oa.splits = (!cta_attn && consumer_merge) ? splits : 0;
    oa.o_part = aa.o_part;
    oa.m_part = aa.m_part;
    oa.l_part = aa.l_part;
    oa.xres_in = xres[0];
    oa.xres_out = xres[1];
    oa.batch = B;
    QUIC_CUDA(launch_oproj(oa, st, true));

    GateUpArgs ga = {};
    ga.w = L.gate_up;
    ga.ln = (const half*)L.ln2;
    ga.xres = xres[1];
    ga.gu_part = gu_part;
    ga.batch = B;
    ga.eps = m->eps;
    QUIC_CUDA(launch_gateup(ga, st, true));

    DownArgs da = {};
    da.w = L.down;
    da.gu_part = gu_part;
    da.partial = partial;
    da.batch = B;
    QUIC_CUDA(launch_down(da, st, true));
  }

  LmHeadArgs la = {};
  la.embed = (const half*)m->embed;
  la.ln = (const half*)m->final_norm;
  la.xres_in = xres[1];
  la.partial = partial;
  la.batch = B;
  la.vocab = m->vocab;
  la.eps = m->eps;
  la.logits = (half*)d->logits;
  la.best_val = reinterpret_cast<float*>(base + ar.best_val);
  la.best_idx = reinterpret_cast<int32_t*>(base + ar.best_idx);
  la.counter = reinterpret_cast<int32_t*>(base + ar.lm_counter);
  la.keys = reinterpret_cast<unsigned long long*>(base + ar.lm_counter + 256);
  la.rows = d->rows;
  la.tok = d->tok;
  la.pos = d->pos;
  la.out_tokens = d->out_tokens;
  la.n_slots = d->n_slots;
  la.ring = d->ring > 0 ? d->ring : 1;
  la.step_counter = d->step_counter;
  QUIC_CUDA(launch_lm_head(la, lm_head_grid(m->vocab), st, true));
  return QUIC_OK;
}

// 2..16 rows: five launches per layer as for one row, every linear on mma.sync with the rows on
// the M side; each kernel writes a finished fp16 tensor (decode_layers_mma.cu).
int enqueue_step_rows16(const quic_model_t* m, const quic_decode_t* d, cudaStream_t st, bool chain_head) {
  const int B = d->batch;
  const int splits = pick_splits(d);
  const Arena ar = carve(B, m->vocab, splits);
  char* base = static_cast<char*>(d->scratch);
  half* xa = reinterpret_cast<half*>(base + ar.xres);  // residual stream entering a layer
  half* xb = xa + (size_t)B * kHidden;                  // after the attention block
  half* qbuf = reinterpret_cast<half*>(base + ar.qbuf);
  half* attn_out = reinterpret_cast<half*>(base + ar.attn_out);
  half* act = reinterpret_cast<half*>(base + ar.act16);
  half* xn = reinterpret_cast<half*>(base + ar.xn);
  // per-tile sums of squares of the two residual streams ([B][32] fp32 each), the down
  // kernel's K-split planes and its arrival counters (in the arena's zeroed head)
  float* ssq_a = reinterpret_cast<float*>(base + ar.act);
  float* ssq_b = ssq_a + kMmaChainMaxRows * 32;
  float* partial = reinterpret_cast<float*>(base + ar.partial);
  int32_t* down_counters = reinterpret_cast<int32_t*>(base + ar.lm_counter + 128);
  const size_t slot_stride = (size_t)kKvHeads * d->s_max * kHeadDim;
  const size_t kv_plane = (size_t)d->n_slots * slot_stride;
  int ctx = d->ctx_hint > 0 ? d->ctx_hint : d->s_max;
  if (ctx > d->s_max) ctx = d->s_max;
  RowState rs;
  rs.rows = d->rows;
  rs.tok = d->tok;
  rs.pos = d->pos;
  rs.batch = B;
  const half* embed = (const half*)m->embed;

  for (int l = 0; l < m->n_layers; ++l) {
    const quic_layer_t& L = m->layers[l];
    half* kc = static_cast<half*>(d->kv) + (size_t)(2 * l) * kv_plane;
    half* vc = kc + kv_plane;
    // (the head of a sequence starts only after everything enqueued before it has completed)
    QUIC_CUDA(launch_qkv_mma(L.qkv, (const half*)L.ln1, embed, xa, ssq_a, xa, rs, m->eps, l == 0, m->vocab,
                             (const half*)m->rope_cos, (const half*)m->rope_sin, m->max_pos, qbuf, kc, vc, d->s_max,
                             st, !(chain_head && l == 0)));
    AttnArgs aa = {};
    aa.q = qbuf;
    aa.k = kc;
    aa.v = vc;
    aa.stride_b = (int64_t)slot_stride;
    aa.stride_h = (int64_t)d->s_max * kHeadDim;
    aa.rows = d->rows;
    aa.pos = d->pos;
    aa.s_cap = ctx;
    aa.splits = splits;
    aa.chunk = (ctx + splits - 1) / splits;
    aa.scale = 0.125f;
    aa.out = attn_out;
    aa.small = (splits <= 32 && (int64_t)splits * 64 >= ctx) ? 1 : 0;
    aa.use_mma = 1;
    aa.consumer_merge = 0;  // the splits are merged by the last CTA to arrive
    aa.epoch = d->step_counter;
    aa.prefetch = (aa.small && d->step_counter != nullptr) ? 1 : 0;
    if (attn_cta_splits(ctx) <= kAttnCtaMaxSplits) {
      // up to 4096 tokens: CTAs of 512 tokens, merged through (distributed) shared memory
      aa.splits = attn_cta_splits(ctx);
      aa.chunk = 512;
      aa.prefetch = d->step_counter != nullptr ? 1 : 0;
      QUIC_CUDA(launch_attn_cta(aa, B, st, true));
    } else {
      if (splits > 1) attn_carve_scratch(base + ar.attn, B, splits, &aa);
      QUIC_CUDA(launch_attn(aa, B, st, true));
    }
    QUIC_CUDA(launch_oproj_mma(L.o, attn_out, xa, xb, ssq_b, B, st));
    QUIC_CUDA(launch_gateup_mma(L.gate_up, (const half*)L.ln2, xb, ssq_b, act, B, m->eps, st));
    QUIC_CUDA(launch_down_mma(L.down, act, xb, xa, ssq_a, partial, down_counters, B, st));
  }
  LmHeadArgs la = {};
  la.embed = embed;
  la.batch = B;
  la.vocab = m->vocab;
  la.eps = m->eps;
  la.logits = (half*)d->logits;
  la.best_val = reinterpret_cast<float*>(base + ar.best_val);
  la.best_idx = reinterpret_cast<int32_t*>(base + ar.best_idx);
  la.counter = reinterpret_cast<int32_t*>(base + ar.lm_counter);
  la.keys = reinterpret_cast<unsigned long long*>(base + ar.lm_counter + 256);
  la.rows = d->rows;
  la.tok = d->tok;
  la.pos = d->pos;
  la.out_tokens = d->out_tokens;
  la.n_slots = d->n_slots;
  la.ring = d->ring > 0 ? d->ring : 1;
  la.step_counter = d->step_counter;
  if (B > 4 && lm_head_tc_supported(B, m->vocab)) {
    QUIC_CUDA(launch_rmsnorm(xa, nullptr, (const half*)m->final_norm, m->eps, xn, nullptr, B, st));
    la.x_normed = xn;
    return launch_lm_head_tc(la, st);
  }
  // up to four rows: the GEMV form, final norm fused, one launch
  la.ln = (const half*)m->final_norm;
  la.xres_in = xa;
  QUIC_CUDA(launch_lm_head(la, lm_head_grid(m->vocab), st, true));
  return QUIC_OK;
}

// Batch > 16: every linear is the tcgen05 GEMM; norms, RoPE/KV append and SwiGLU are
// separate small kernels (at these sizes each kernel does microseconds of real work, so
// the launch chain is no longer what bounds the step).
// Up to 20 rows the cluster kernel, whose tiles are requested before the dependency wait (17 rows of
// 200..1500 tokens: 791 us per step against 865 streamed; 24 rows: 963 against 872).
constexpr int kCtaAttnMaxRows = 20;
// One CTA per (row, KV head) is a serial walk over the row: with few rows and very long rows the
// split kernel, which spreads a row over many CTAs, wins (us per step, streamed / split: 24 rows of
// 4000..8000 tokens 1430 / 1555, of 8000..16000 2157 / 1822; 64 rows of 16000..32000 4079 / 4598).
constexpr int kStreamMaxCtx = 8192;
constexpr int kStreamAnyCtxRows = 48;

// `fuse`: the attention kernel finishes the QKV linear itself (only where attention_streams()).
int enqueue_attention(const quic_decode_t* d, const Arena& ar, int splits, int ctx, half* qbuf, half* kc, half* vc,
                      half* attn_out, cudaStream_t st, const QkvFinish* fuse = nullptr);

// More than kCtaAttnMaxRows rows of moderate length: the streamed attention kernel.
bool attention_streams(int batch, int ctx) {
  return batch > kCtaAttnMaxRows && (ctx <= kStreamMaxCtx || batch >= kStreamAnyCtxRows);
}

int enqueue_step_batched(const quic_model_t* m, const quic_decode_t* d, cudaStream_t st, bool chain_head) {
  const int B = d->batch;
  const int splits = pick_splits(d);
  const Arena ar = carve(B, m->vocab, splits);
  char* base = static_cast<char*>(d->scratch);
  half* h = reinterpret_cast<half*>(base + ar.xres);        // residual stream
  half* qbuf = reinterpret_cast<half*>(base + ar.qbuf);
  half* attn_out = reinterpret_cast<half*>(base + ar.attn_out);
  half* xn = reinterpret_cast<half*>(base + ar.xn);
  half* act = reinterpret_cast<half*>(base + ar.act16);
  float* ws = reinterpret_cast<float*>(base + ar.tcws);
  const size_t slot_stride = (size_t)kKvHeads * d->s_max * kHeadDim;
  const size_t kv_plane = (size_t)d->n_slots * slot_stride;
  int ctx = d->ctx_hint > 0 ? d->ctx_hint : d->s_max;
  if (ctx > d->s_max) ctx = d->s_max;
  const half* embed = (const half*)m->embed;

  // (the head of a sequence starts only after everything enqueued before it has completed)
  QUIC_CUDA(launch_embed_rows(embed, d->rows, d->tok, m->vocab, h, B, st, !chain_head));
  QUIC_CUDA(launch_rmsnorm(h, nullptr, (const half*)m->layers[0].ln1, m->eps, xn, nullptr, B, st));
  for (int l = 0; l < m->n_layers; ++l) {
    const quic_layer_t& L = m->layers[l];
    half* kc = static_cast<half*>(d->kv) + (size_t)(2 * l) * kv_plane;
    half* vc = kc + kv_plane;
    // linears whose consumer is a small kernel leave split-K partials for it to reduce
    int sp = 1;
    const float* part = ws + 4096;
    int rc = w4a16_gemm_tc(xn, L.qkv, nullptr, B, ws, st, &sp);
    if (rc != QUIC_OK) return rc;
    if (attention_streams(B, ctx)) {
      // the attention CTAs sum the partial sums, rotate and append themselves: one launch less
      // (64 rows of 512 tokens: 934 -> 883 us per step, same bits)
      QkvFinish fin = {part, sp, (const half*)L.qkv.bias, nullptr, (const half*)m->rope_cos, (const half*)m->rope_sin,
                       m->max_pos};
      rc = enqueue_attention(d, ar, splits, ctx, qbuf, kc, vc, attn_out, st, &fin);
    } else {
      QUIC_CUDA(launch_qkv_post_part(part, sp, (const half*)L.qkv.bias, d->rows, d->pos, (const half*)m->rope_cos,
                                     (const half*)m->rope_sin, m->max_pos, qbuf, kc, vc, d->s_max, d->n_slots, B, st));
      rc = enqueue_attention(d, ar, splits, ctx, qbuf, kc, vc, attn_out, st);
    }
    if (rc != QUIC_OK) return rc;
    rc = w4a16_gemm_tc(attn_out, L.o, nullptr, B, ws, st, &sp);
    if (rc != QUIC_OK) return rc;
    QUIC_CUDA(launch_rmsnorm_part(part, sp, h, (const half*)L.ln2, m->eps, xn, h, B, st));
    rc = w4a16_gemm_tc_swiglu(xn, L.gate_up, act, B, st);  // SwiGLU in the GEMM's epilogue
    if (rc != QUIC_OK) return rc;
    rc = w4a16_gemm_tc(act, L.down, nullptr, B, ws, st, &sp);
    if (rc != QUIC_OK) return rc;
    const half* next_ln = (l + 1 < m->n_layers) ? (const half*)m->layers[l + 1].ln1 : (const half*)m->final_norm;
    QUIC_CUDA(launch_rmsnorm_part(part, sp, h, next_ln, m->eps, xn, h, B, st));
  }
  LmHeadArgs la = {};
  la.embed = embed;
  la.x_normed = xn;
  la.batch = B;
  la.vocab = m->vocab;
  la.eps = m->eps;
  la.logits = (half*)d->logits;
  la.best_val = reinterpret_cast<float*>(base + ar.best_val);
  la.best_idx = reinterpret_cast<int32_t*>(base + ar.best_idx);
  la.counter = reinterpret_cast<int32_t*>(base + ar.lm_counter);
  la.keys = reinterpret_cast<unsigned long long*>(base + ar.lm_counter + 256);
  la.rows = d->rows;
  la.tok = d->tok;
  la.pos = d->pos;
  la.out_tokens = d->out_tokens;
  la.n_slots = d->n_slots;
  la.ring = d->ring > 0 ? d->ring : 1;
  la.step_counter = d->step_counter;
  if (lm_head_tc_supported(B, m->vocab)) return launch_lm_head_tc(la, st);
  la.x_normed = xn;
  QUIC_CUDA(launch_lm_head(la, lm_head_grid(m->vocab), st, false));
  return QUIC_OK;
}

// Attention of a decode step with finished fp16 output: the scratch-free CTA form up to 4096
// tokens and 32 rows, the split form merged by the last CTA to arrive beyond.
int enqueue_attention(const quic_decode_t* d, const Arena& ar, int splits, int ctx, half* qbuf, half* kc, half* vc,
                      half* attn_out, cudaStream_t st, const QkvFinish* fuse) {
  const int B = d->batch;
  char* base = static_cast<char*>(d->scratch);
  const size_t slot_stride = (size_t)kKvHeads * d->s_max * kHeadDim;
  AttnArgs aa = {};
  aa.q = qbuf;
  aa.k = kc;
  aa.v = vc;
  aa.stride_b = (int64_t)slot_stride;
  aa.stride_h = (int64_t)d->s_max * kHeadDim;
  aa.rows = d->rows;
  aa.pos = d->pos;
  aa.s_cap = ctx;
  aa.scale = 0.125f;  // 64^-0.5, src/model.py:129
  aa.out = attn_out;
  aa.use_mma = 1;
  aa.consumer_merge = 0;
  aa.epoch = d->step_counter;
  // few rows: CTAs of 512 tokens, clusters beyond, no scratch
  if (attn_cta_splits(ctx) <= kAttnCtaMaxSplits && B <= kCtaAttnMaxRows) {
    aa.splits = attn_cta_splits(ctx);
    aa.chunk = 512;
    aa.prefetch = d->step_counter != nullptr ? 1 : 0;
    QUIC_CUDA(launch_attn_cta(aa, B, st, true));
    return QUIC_OK;
  }
  if (attention_streams(B, ctx)) {
    // more rows: one CTA per (row, KV head) streams the row's cache through a TMA ring
    // (64 rows of 200..1500 tokens: 1266 -> 1015 us per step; of 512: 1050 -> 924; of 2000..4000: 1622 -> 1307)
    aa.splits = 1;
    aa.chunk = ctx;
    aa.prefetch = d->step_counter != nullptr ? 1 : 0;
    return launch_attn_stream(aa, fuse, B, d->n_slots, d->s_max, tc_status_words(), st, true);
  }
  aa.splits = splits;
  aa.chunk = (ctx + splits - 1) / splits;
  aa.small = (splits <= 32 && (int64_t)splits * 64 >= ctx) ? 1 : 0;
  aa.prefetch = (aa.small && d->step_counter != nullptr) ? 1 : 0;
  if (splits > 1) attn_carve_scratch(base + ar.attn, B, splits, &aa);
  QUIC_CUDA(launch_attn(aa, B, st, true));
  return QUIC_OK;
}

LmHeadArgs lm_head_args(const quic_model_t* m, const quic_decode_t* d, const Arena& ar) {
  char* base = static_cast<char*>(d->scratch);
  LmHeadArgs la = {};
  la.embed = (const half*)m->embed;
  la.batch = d->batch;
  la.vocab = m->vocab;
  la.eps = m->eps;
  la.logits = (half*)d->logits;
  la.best_val = reinterpret_cast<float*>(base + ar.best_val);
  la.best_idx = reinterpret_cast<int32_t*>(base + ar.best_idx);
  la.counter = reinterpret_cast<int32_t*>(base + ar.lm_counter);
  la.keys = reinterpret_cast<unsigned long long*>(base + ar.lm_counter + 256);
  la.rows = d->rows;
  la.tok = d->tok;
  la.pos = d->pos;
  la.out_tokens = d->out_tokens;
  la.n_slots = d->n_slots;
  la.ring = d->ring > 0 ? d->ring : 1;
  la.step_counter = d->step_counter;
  return la;
}

// Dense fp16 weights, one or two rows: five kernels per layer (decode_layers_f16.cu) and the GEMV
// lm_head with the final norm fused.
int enqueue_step_f16(const quic_model_t* m, const quic_decode_t* d, cudaStream_t st, bool chain_head) {
  const int B = d->batch;
  const int splits = pick_splits(d);
  const Arena ar = carve(B, m->vocab, splits);
  char* base = static_cast<char*>(d->scratch);
  half* xa = reinterpret_cast<half*>(base + ar.xres);  // residual stream entering a layer
  half* xb = xa + (size_t)B * kHidden;                  // after the attention block
  half* qbuf = reinterpret_cast<half*>(base + ar.qbuf);
  half* attn_out = reinterpret_cast<half*>(base + ar.attn_out);
  half* act = reinterpret_cast<half*>(base + ar.act);
  const size_t kv_plane = (size_t)d->n_slots * kKvHeads * d->s_max * kHeadDim;
  int ctx = d->ctx_hint > 0 ? d->ctx_hint : d->s_max;
  if (ctx > d->s_max) ctx = d->s_max;
  RowState rs;
  rs.rows = d->rows;
  rs.tok = d->tok;
  rs.pos = d->pos;
  rs.batch = B;
  for (int l = 0; l < m->n_layers; ++l) {
    const quic_layer_t& L = m->layers[l];
    half* kc = static_cast<half*>(d->kv) + (size_t)(2 * l) * kv_plane;
    half* vc = kc + kv_plane;
    QUIC_CUDA(launch_qkv_f16(L.qkv, (const half*)L.ln1, (const half*)m->embed, xa, xa, rs, m->eps, l == 0, m->vocab,
                             (const half*)m->rope_cos, (const half*)m->rope_sin, m->max_pos, qbuf, kc, vc, d->s_max,
                             d->n_slots, st, !(chain_head && l == 0)));
    int rc = enqueue_attention(d, ar, splits, ctx, qbuf, kc, vc, attn_out, st);
    if (rc != QUIC_OK) return rc;
    QUIC_CUDA(launch_residual_f16(L.o, attn_out, xa, xb, B, st));
    QUIC_CUDA(launch_gateup_f16(L.gate_up, (const half*)L.ln2, xb, act, B, m->eps, st));
    QUIC_CUDA(launch_residual_f16(L.down, act, xb, xa, B, st));
  }
  LmHeadArgs la = lm_head_args(m, d, ar);
  la.ln = (const half*)m->final_norm;
  la.xres_in = xa;
  QUIC_CUDA(launch_lm_head(la, lm_head_grid(m->vocab), st, true));
  return QUIC_OK;
}

// Dense fp16 weights, more rows: every linear on the tcgen05 fp16 GEMM; norms, RoPE / KV append
// and SwiGLU are the small kernels of the batched W4A16 step.
int enqueue_step_batched_f16(const quic_model_t* m, const quic_decode_t* d, cudaStream_t st, bool chain_head) {
  const int B = d->batch;
  const int splits = pick_splits(d);
  const Arena ar = carve(B, m->vocab, splits);
  char* base = static_cast<char*>(d->scratch);
  half* h = reinterpret_cast<half*>(base + ar.xres);
  half* qbuf = reinterpret_cast<half*>(base + ar.qbuf);
  half* attn_out = reinterpret_cast<half*>(base + ar.attn_out);
  half* xn = reinterpret_cast<half*>(base + ar.xn);
  half* qkv = reinterpret_cast<half*>(base + ar.qkv);  // [B][1152]; also holds a [B][896] linear output
  half* gu = reinterpret_cast<half*>(base + ar.gu);
  half* act = reinterpret_cast<half*>(base + ar.act16);
  float* ws = reinterpret_cast<float*>(base + ar.tcws);  // split-K partials of the small GEMMs
  const size_t kv_plane = (size_t)d->n_slots * kKvHeads * d->s_max * kHeadDim;
  int ctx = d->ctx_hint > 0 ? d->ctx_hint : d->s_max;
  if (ctx > d->s_max) ctx = d->s_max;
  QUIC_CUDA(launch_embed_rows((const half*)m->embed, d->rows, d->tok, m->vocab, h, B, st, !chain_head));
  QUIC_CUDA(launch_rmsnorm(h, nullptr, (const half*)m->layers[0].ln1, m->eps, xn, nullptr, B, st));
  for (int l = 0; l < m->n_layers; ++l) {
    const quic_layer_t& L = m->layers[l];
    half* kc = static_cast<half*>(d->kv) + (size_t)(2 * l) * kv_plane;
    half* vc = kc + kv_plane;
    int rc = gemm_f16_tc(xn, (const half*)L.qkv.w16, (const half*)L.qkv.bias, qkv, B, kQkvN, kHidden, ws, st, true);
    if (rc != QUIC_OK) return rc;
    if (attention_streams(B, ctx)) {  // the attention CTAs rotate and append themselves
      QkvFinish fin = {nullptr, 0, nullptr, qkv, (const half*)m->rope_cos, (const half*)m->rope_sin, m->max_pos};
      rc = enqueue_attention(d, ar, splits, ctx, qbuf, kc, vc, attn_out, st, &fin);
    } else {
      QUIC_CUDA(launch_qkv_post(qkv, d->rows, d->pos, (const half*)m->rope_cos, (const half*)m->rope_sin, m->max_pos,
                                qbuf, kc, vc, d->s_max, d->n_slots, B, st));
      rc = enqueue_attention(d, ar, splits, ctx, qbuf, kc, vc, attn_out, st);
    }
    if (rc != QUIC_OK) return rc;
    rc = gemm_f16_tc(attn_out, (const half*)L.o.w16, nullptr, qkv, B, kHidden, kHidden, ws, st, true);
    if (rc != QUIC_OK) return rc;
    QUIC_CUDA(launch_rmsnorm(qkv, h, (const half*)L.ln2, m->eps, xn, h, B, st));
    rc = gemm_f16_tc(xn, (const half*)L.gate_up.w16, nullptr, gu, B, 2 * kInter, kHidden, ws, st, true);
    if (rc != QUIC_OK) return rc;
    QUIC_CUDA(launch_swiglu_fused(gu, act, B, st));
    rc = gemm_f16_tc(act, (const half*)L.down.w16, nullptr, qkv, B, kHidden, kInter, ws, st, true);
    if (rc != QUIC_OK) return rc;
    const half* next_ln = (l + 1 < m->n_layers) ? (const half*)m->layers[l + 1].ln1 : (const half*)m->final_norm;
    QUIC_CUDA(launch_rmsnorm(qkv, h, next_ln, m->eps, xn, h, B, st));
  }
  LmHeadArgs la = lm_head_args(m, d, ar);
  la.x_normed = xn;
  if (lm_head_tc_supported(B, m->vocab)) return launch_lm_head_tc(la, st);
  QUIC_CUDA(launch_lm_head(la, lm_head_grid(m->vocab), st, false));
  return QUIC_OK;
}

struct Graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  bool tensor_kernels = false;  // the step holds tcgen05 kernels, whose bounded waits report through error words
};

}  // namespace
}  // namespace quic

using namespace quic;

extern "C" void quic_set_tensor_min_batch(int32_t batch) {
  g_tensor_min_batch = batch < 2 ? 2 : (batch > kMmaChainMaxRows + 1 ? kMmaChainMaxRows + 1 : batch);
}

extern "C" void quic_set_mma_chain_min_batch(int32_t batch) {
  g_mma_chain_min_batch = batch < 2 ? 2 : (batch > kMmaChainMaxRows + 1 ? kMmaChainMaxRows + 1 : batch);
}

extern "C" int32_t quic_decode_pick_splits(int32_t batch, int32_t ctx) {
  if (batch < 1) batch = 1;
  if (ctx < 1) ctx = 1;
  // Throughput regime (tensor-core step): 4-warp CTAs that cover 128 tokens per pass; one
  // pass per CTA while that still leaves at most two waves of four CTAs per SM.
  if (batch >= g_tensor_min_batch) {
    if (ctx <= 2048) return (ctx + 63) / 64;  // single-warp CTAs, every cache tile in flight at once
    const int by_len = (ctx + 127) / 128;
    int s = 1184 / (batch * kKvHeads);
    if (s > by_len) s = by_len;
    if (s > 64) s = 64;
    return s < 1 ? 1 : s;
  }
  // Up to 2048 tokens at small batch: one warp per 64 tokens, merged by the o_proj kernel.
  const int small = (ctx + 63) / 64;
  if (small <= kWarpMaxSplits) return small;
  // Longer: 4-warp CTAs of the throughput kernel over 128 tokens and more each, and no more
  // splits than the o_proj kernel merges itself.
  const int by_len = (ctx + 127) / 128;
  return by_len < kMaxConsumerSplitsTotal ? by_len : kMaxConsumerSplitsTotal;
}

extern "C" int64_t quic_decode_scratch_bytes(int32_t batch, int32_t vocab, int32_t attn_splits) {
  if (batch < 1 || vocab < 2 || attn_splits < 1) return 0;
  return carve(batch, vocab, attn_splits).total;
}

extern "C" int32_t quic_decode_launch_count(const quic_model_t* m, const quic_decode_t* d) {
  if (!m) return 0;
  if (m->layers && m->layers[0].qkv.w16 != nullptr) {
    if (d && d->batch > kF16ChainMaxRows) {
      int ctx = d->ctx_hint > 0 ? d->ctx_hint : d->s_max;
      if (ctx > d->s_max) ctx = d->s_max;
      return (attention_streams(d->batch, ctx) ? 8 : 9) * m->n_layers + 3;
    }
    return 5 * m->n_layers + 1;
  }
  if (d && d->batch >= g_tensor_min_batch) {
    int ctx = d->ctx_hint > 0 ? d->ctx_hint : d->s_max;
    if (ctx > d->s_max) ctx = d->s_max;
    return (attention_streams(d->batch, ctx) ? 7 : 8) * m->n_layers + 3;  // the streamed attention finishes the QKV linear
  }
  if (d && d->batch >= g_mma_chain_min_batch) return 5 * m->n_layers + ((d->batch > 4 && lm_head_tc_supported(d->batch, m->vocab)) ? 2 : 1);
  return 5 * m->n_layers + 1;
}

extern "C" int quic_decode_step(const quic_model_t* m, const quic_decode_t* d, void* stream) {
  int rc = check(m, d);
  if (rc != QUIC_OK) return rc;
  return enqueue_step(m, d, (cudaStream_t)stream, true);
}

extern "C" int quic_decode_graph_create(const quic_model_t* m, const quic_decode_t* d,
                                        int32_t steps, void* stream, void** graph_out) {
  int rc = check(m, d);
  if (rc != QUIC_OK) return rc;
  QUIC_REQUIRE(graph_out != nullptr && steps >= 1 && steps <= 4096, QUIC_E_ARG,
               "decode_graph_create: bad steps / output pointer");
  cudaStream_t st = (cudaStream_t)stream;
  QUIC_REQUIRE(st != nullptr, QUIC_E_ARG,
               "decode_graph_create: capture needs a non-default stream");
  Graph* g = new (std::nothrow) Graph();
  QUIC_REQUIRE(g != nullptr, QUIC_E_ARG, "decode_graph_create: out of host memory");
  cudaError_t e = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
  if (e != cudaSuccess) {
    delete g;
    return fail(QUIC_E_CUDA, cudaGetErrorString(e));
  }
  for (int s = 0; s < steps && rc == QUIC_OK; ++s) rc = enqueue_step(m, d, st, s == 0);
  e = cudaStreamEndCapture(st, &g->graph);
  if (rc == QUIC_OK && e != cudaSuccess) rc = fail(QUIC_E_CUDA, cudaGetErrorString(e));
  if (rc == QUIC_OK) {
    e = cudaGraphInstantiate(&g->exec, g->graph, 0);
    if (e != cudaSuccess) rc = fail(QUIC_E_CUDA, cudaGetErrorString(e));
  }
  if (rc != QUIC_OK) {
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
    cudaGetLastError();
    return rc;
  }
  const bool dense = m->layers[0].qkv.w16 != nullptr;
  g->tensor_kernels = dense ? d->batch > kF16ChainMaxRows
                            : (d->batch >= g_tensor_min_batch ||
                               (d->batch >= g_mma_chain_min_batch && d->batch > 4 && lm_head_tc_supported(d->batch, m->vocab)));
  *graph_out = g;
  return QUIC_OK;
}

extern "C" int quic_graph_launch(void* graph, void* stream) {
  QUIC_REQUIRE(graph != nullptr, QUIC_E_ARG, "graph_launch: null graph");
  Graph* g = static_cast<Graph*>(graph);
  QUIC_CUDA(cudaGraphLaunch(g->exec, (cudaStream_t)stream));
  return QUIC_OK;
}

extern "C" int quic_graph_run_host(void* graph, void* stream, const int32_t* host_in, int32_t* dev_in,
                                   int32_t n_in, const int32_t* dev_out, int32_t* host_out, int32_t n_out) {
  QUIC_REQUIRE(graph != nullptr, QUIC_E_ARG, "graph_run_host: null graph");
  QUIC_REQUIRE(n_in >= 0 && n_out >= 0, QUIC_E_ARG, "graph_run_host: negative count");
  QUIC_REQUIRE(n_in == 0 || (host_in != nullptr && dev_in != nullptr), QUIC_E_ARG,
               "graph_run_host: null input buffer");
  QUIC_REQUIRE(n_out == 0 || (host_out != nullptr && dev_out != nullptr), QUIC_E_ARG,
               "graph_run_host: null output buffer");
  Graph* g = static_cast<Graph*>(graph);
  cudaStream_t st = (cudaStream_t)stream;
  if (n_in > 0) QUIC_CUDA(cudaMemcpyAsync(dev_in, host_in, sizeof(int32_t) * n_in, cudaMemcpyHostToDevice, st));
  QUIC_CUDA(cudaGraphLaunch(g->exec, st));
  if (n_out > 0)
    QUIC_CUDA(cudaMemcpyAsync(host_out, dev_out, sizeof(int32_t) * n_out, cudaMemcpyDeviceToHost, st));
  // the error words of the tensor-core kernels ride along with the tokens (the GEMV and mma.sync
  // chains hold no kernel that waits on a barrier: nothing to ask for)
  if (g->tensor_kernels) {
    const int rc = tc_status_poll_async(st);
    if (rc != QUIC_OK) return rc;
  }
  QUIC_CUDA(cudaStreamSynchronize(st));
  const int word = g->tensor_kernels ? tc_status_polled(st) : 0;
  if (word != 0) {
    static char msg[160];
    snprintf(msg, sizeof(msg),
             "decode: a bounded wait of a tensor-core kernel gave up (status 0x%x); the tokens of this call are invalid",
             word);
    return fail(QUIC_E_TIMEOUT, msg);
  }
  return QUIC_OK;
}

extern "C" int quic_graph_destroy(void* graph) {
  if (graph == nullptr) return QUIC_OK;
  Graph* g = static_cast<Graph*>(graph);
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  delete g;
  return QUIC_OK;
}
