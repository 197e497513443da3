// Kernel argument blocks and launchers of the fused decode step.
#pragma once
#include "common.cuh"

namespace quic {

// Rows of the down-projection split over kDownSplits CTAs along K (38 groups).
constexpr int kDownSplits = 5;
__host__ __device__ __forceinline__ int down_group_begin(int ks) {
  // 8,8,8,7,7 groups
  return ks <= 3 ? ks * 8 : 24 + (ks - 3) * 7;
}
constexpr int kMaxM = 8;  // batch rows per CTA pass
// The o_proj kernel merges the attention splits itself: this many per pass of loads, up to
// kMaxConsumerSplitsTotal in all.  kWarpMaxSplits: the single-warp attention kernel covers a
// context of up to this many 64-token tiles (2048 tokens).
constexpr int kMaxConsumerSplits = 16;
constexpr int kMaxConsumerSplitsTotal = 64;
constexpr int kWarpMaxSplits = 32;

struct RowState {
  const int32_t* rows;  // [batch] slot per row
  const int32_t* tok;   // [n_slots]
  const int32_t* pos;   // [n_slots]
  int32_t batch;
};

struct QkvArgs {
  quic_w4_t w;
  const half* ln;
  const half* embed;      // used when first_layer
  const half* xres_in;    // [batch][896]
  half* xres_out;         // [batch][896]
  const float* partial;   // [kDownSplits][batch][896] or nullptr (first layer)
  RowState rs;
  float eps;
  int32_t first_layer;
  int32_t vocab;
  const half* cos_t;
  const half* sin_t;
  int32_t max_pos;
  half* qbuf;    // [batch][14][64]
  half* kcache;  // this layer: [n_slots][2][s_max][64]
  half* vcache;
  int32_t s_max;
};

struct OProjArgs {
  quic_w4_t w;
  // splits > 0: merge the attention kernel's split partials here
  int32_t splits;
  const float* o_part;  // [batch][14][splits][64]
  const float* m_part;  // [batch][14][splits]
  const float* l_part;
  const half* attn;     // [batch][896] (splits == 0)
  const half* xres_in;  // [batch][896]
  half* xres_out;
  int32_t batch;
};

struct GateUpArgs {
  quic_w4_t w;  // n = 9728
  const half* ln;
  const half* xres;  // [batch][896]
  float* gu_part;    // [2 parts][gate|up][batch][4864] fp32 partial sums
  int32_t batch;
  float eps;
};

struct DownArgs {
  quic_w4_t w;
  const float* gu_part;  // [2 parts][gate|up][batch][4864]
  float* partial;        // [kDownSplits][batch][896]
  int32_t batch;
};

struct AttnArgs {
  const half* q;  // [batch][14][64]
  const half* k;
  const half* v;
  int64_t stride_b;  // elements between slots / batch rows
  int64_t stride_h;  // elements between kv heads
  const int32_t* start;  // [batch] or nullptr
  const int32_t* end;    // [batch] or nullptr
  const int32_t* rows;   // decode-step mode: slot per row, end = pos[slot]+1
  const int32_t* pos;
  int32_t s_cap;  // token range covered by the grid
  int32_t chunk;  // tokens per split
  int32_t splits;
  int32_t consumer_merge;  // 1: write partials only, the o_proj kernel merges
  int32_t small;           // 1: latency variant (one warp per 64 tokens)
  int32_t prefetch;        // latency variant inside the decode chain: cache tile requested before the wait
  const int32_t* epoch;    // step counter that guards the early request (advanced once per decode step)
  int32_t use_mma;         // 1: throughput variant on mma.m16n8k16
  float scale;
  half* out;  // [batch][896]
  int32_t* counters;  // [batch][2]
  float* o_part;      // [batch][14][splits][64]
  float* m_part;      // [batch][14][splits]
  float* l_part;
};

// Scratch-free attention (attn_decode_cta.cu): CTAs of 512 tokens, a.splits of them (a cluster)
// per (row, KV head).
constexpr int kAttnCtaMaxSplits = 8;
int attn_cta_splits(int ctx);
cudaError_t launch_attn_cta(const AttnArgs& a, int batch, cudaStream_t stream, bool pdl);
// Many rows: one CTA per (row, KV head) streaming the cache through a TMA ring (attn_decode_stream.cu).
// `fuse` (or nullptr): the kernel also finishes the fused QKV linear for its row -- sums the split-K
// partial sums, adds the bias, rotates q and k, appends k and v to the cache -- so that no separate
// kernel stands between the QKV GEMM and the attention.
struct QkvFinish {
  const float* part;  // [splits][batch][1152] fp32 partial sums of the QKV linear (columns in the prepacked order)
  int32_t splits;
  const half* bias;   // [1152]
  const half* qkv;    // instead of part / splits / bias: the linear's finished fp16 output [batch][1152]
  const half* cos_t;  // [max_pos][32]
  const half* sin_t;
  int32_t max_pos;
};
int launch_attn_stream(const AttnArgs& a, const QkvFinish* fuse, int batch, int n_slots, int s_max, int* status,
                       cudaStream_t stream, bool pdl);

struct LmHeadArgs {
  const half* embed;  // [vocab][896]
  const half* ln;
  const half* xres_in;   // [batch][896]
  const float* partial;  // [kDownSplits][batch][896] or nullptr
  const half* x_normed;  // stand-alone GEMV mode: rows already normalised, or nullptr
  int32_t batch;
  int32_t vocab;
  float eps;
  half* logits;  // [batch][vocab] or nullptr
  // argmax
  float* best_val;    // [batch][grid]
  int32_t* best_idx;  // [batch][grid]
  int32_t* counter;   // single int
  unsigned long long* keys;  // tensor path: [batch] packed (logit, index) maxima, zero when idle
  // state update by the last CTA (all optional)
  const int32_t* rows;
  int32_t* tok;
  int32_t* pos;
  int32_t* out_tokens;
  int32_t n_slots;
  int32_t ring;
  int32_t* step_counter;
  int64_t* argmax_out;  // stand-alone mode: [batch]
};

cudaError_t launch_qkv(const QkvArgs& a, cudaStream_t s, bool pdl);
cudaError_t launch_oproj(const OProjArgs& a, cudaStream_t s, bool pdl);
cudaError_t launch_gateup(const GateUpArgs& a, cudaStream_t s, bool pdl);
cudaError_t launch_down(const DownArgs& a, cudaStream_t s, bool pdl);
cudaError_t launch_attn(const AttnArgs& a, int batch, cudaStream_t s, bool pdl);
cudaError_t launch_lm_head(const LmHeadArgs& a, int grid, cudaStream_t s, bool pdl);
int lm_head_grid(int vocab);

// the layer kernels for 2..16 rows (decode_layers_mma.cu)
constexpr int kMmaChainMaxRows = 16;
cudaError_t launch_qkv_mma(const quic_w4_t& w, const half* ln, const half* embed, const half* x_in,
                           const float* ssq_in, half* x_copy, const RowState& rs, float eps, bool first_layer,
                           int vocab, const half* cos_t, const half* sin_t, int max_pos, half* qbuf, half* kcache,
                           half* vcache, int s_max, cudaStream_t st, bool pdl);
cudaError_t launch_oproj_mma(const quic_w4_t& w, const half* attn, const half* xres_in, half* xres_out, float* ssq_out,
                             int batch, cudaStream_t st);
cudaError_t launch_gateup_mma(const quic_w4_t& w, const half* ln, const half* xres, const float* ssq_in, half* act,
                              int batch, float eps, cudaStream_t st);
cudaError_t launch_down_mma(const quic_w4_t& w, const half* act, const half* xres_in, half* xres_out, float* ssq_out,
                            float* partial, int32_t* counters, int batch, cudaStream_t st);

// Dense fp16 weights (quic_w4_t.w16): the layer chain for 1..kF16ChainMaxRows rows
// (decode_layers_f16.cu) and the tcgen05 GEMM for more rows and for prefill (gemm_f16_tc.cu).
constexpr int kF16ChainMaxRows = 2;  // measured: 493 / 593 us per step at 1 / 2 rows, ~890 us on the GEMM step from 3
cudaError_t launch_qkv_f16(const quic_w4_t& w, const half* ln, const half* embed, const half* x_in, half* x_copy,
                           const RowState& rs, float eps, bool first_layer, int vocab, const half* cos_t,
                           const half* sin_t, int max_pos, half* qbuf, half* kcache, half* vcache, int s_max,
                           int n_slots, cudaStream_t st, bool pdl);
cudaError_t launch_residual_f16(const quic_w4_t& w, const half* x, const half* xres_in, half* xres_out, int batch,
                                cudaStream_t st);
cudaError_t launch_gateup_f16(const quic_w4_t& w, const half* ln, const half* xres, half* act, int batch, float eps,
                              cudaStream_t st);
bool gemm_f16_tc_supported(int m, int n, int k);
int64_t gemm_f16_tc_workspace(int m, int n, int k);
int gemm_f16_tc(const half* x, const half* w, const half* bias, half* y, int m, int n, int k, float* ws,
                cudaStream_t st, bool pdl);

// pieces of the batched (batch > 8) decode step
cudaError_t launch_embed_rows(const half* embed, const int32_t* rows, const int32_t* tok, int vocab, half* x,
                              int batch, cudaStream_t st, bool pdl);
// Fused consumers of split-K partial sums [splits][batch][N] (fp32).
cudaError_t launch_qkv_post_part(const float* part, int splits, const half* bias, const int32_t* rows,
                                 const int32_t* pos, const half* cos_t, const half* sin_t, int max_pos, half* qbuf,
                                 half* kcache, half* vcache, int s_max, int n_slots, int batch, cudaStream_t st);
cudaError_t launch_rmsnorm_part(const float* part, int splits, const half* residual, const half* w, float eps,
                                half* y, half* sum_out, int rows, cudaStream_t st);
cudaError_t launch_qkv_post(const half* qkv, const int32_t* rows, const int32_t* pos, const half* cos_t,
                            const half* sin_t, int max_pos, half* qbuf, half* kcache, half* vcache, int s_max,
                            int n_slots, int batch, cudaStream_t st);
cudaError_t launch_swiglu_fused(const half* gu, half* act, int batch, cudaStream_t st);
// prefill pieces, chainable with programmatic dependent launch
cudaError_t launch_qkv_rope_append(const half* qkv, const int32_t* slots, const int32_t* positions, const half* cos_t,
                                   const half* sin_t, int max_pos, half* q_out, half* kcache, half* vcache, int s_max,
                                   int n_slots, int rows, cudaStream_t st, bool pdl);
// tcgen05 + TMA form for prompts of 128 tokens and more (attn_prefill_tc.cu)
bool attn_prefill_tc_supported(int n_seq, int max_len, int rows, int s_max, int n_slots);
int attn_prefill_tc_launch(const void* q, const void* kcache, const void* vcache, const int32_t* seq_start,
                           const int32_t* seq_len, const int32_t* seq_slot, const int32_t* seq_off, int32_t n_seq,
                           int32_t max_len, int32_t rows, int32_t s_max, int32_t n_slots, float scale, void* out,
                           cudaStream_t stream, bool pdl);
int attn_prefill_launch(const void* q, const void* kcache, const void* vcache, const int32_t* seq_start,
                        const int32_t* seq_len, const int32_t* seq_slot, const int32_t* seq_off, int32_t n_seq,
                        int32_t max_len, int32_t rows, int32_t s_max, int32_t n_slots, float scale, void* out,
                        cudaStream_t stream, bool pdl);
cudaError_t launch_rmsnorm(const half* x, const half* residual, const half* w, float eps, half* y, half* sum_out,
                           int rows, cudaStream_t st);
int w4a16_gemm_tc(const half* x, const quic_w4_t& w, half* y, int m, float* workspace, cudaStream_t st,
                  int* splits_out = nullptr);
int64_t w4a16_gemm_tc_workspace(int m, int n, int k);
int w4a16_gemm_tc_swiglu(const half* x, const quic_w4_t& w, half* act, int m, cudaStream_t st);
bool lm_head_tc_supported(int batch, int vocab);
int lm_head_tc_tiles(int vocab);
int launch_lm_head_tc(const LmHeadArgs& a, cudaStream_t st);
// Error words of the tcgen05 kernels ([0] GEMM, [1] lm_head; w4_gemm_tc.cu): device address,
// an asynchronous copy to page-locked memory, and the value seen by that copy (taken, i.e.
// exchanged with zero, when it is not 0).
int* tc_status_words();
int tc_status_poll_async(cudaStream_t st);
int tc_status_polled(cudaStream_t st);

}  // namespace quic
