/*
 * quic_b200.h — C ABI of the B200 (sm_100a) W4A16 decode path.
 *
 * Every entry point takes plain device pointers and sizes, launches on the
 * stream handle it is given (a cudaStream_t passed as void*), never
 * synchronises, never allocates device memory, and returns 0 on success or a
 * negative QUIC_E_* code.  quic_last_error() returns a static message for the
 * most recent failure on the calling thread.
 *
 * Each declaration cites the interface of the reference project
 * (hdahroug/quic.cu, paths relative to its root) that it replaces.
 *
 * Model constants are fixed at compile time, as in the reference's kernels
 * (kernels/cuda/rmsnorm.cu:7, swiglu.cu:10, flash_attn_decode.cu:8):
 * hidden 896, 14 query heads, 2 KV heads, head_dim 64, intermediate 4864,
 * quantisation group 128.  Layer count, vocabulary size and cache geometry
 * are run-time arguments.
 */
#ifndef QUIC_B200_H
#define QUIC_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QUIC_HIDDEN 896
#define QUIC_HEADS 14
#define QUIC_KV_HEADS 2
#define QUIC_HEAD_DIM 64
#define QUIC_INTER 4864
#define QUIC_GROUP 128
#define QUIC_QKV_N 1152 /* 896 q + 128 k + 128 v */

#define QUIC_OK 0
#define QUIC_E_ARG (-1)     /* bad pointer, size or alignment */
#define QUIC_E_SHAPE (-2)   /* shape not supported by the kernels */
#define QUIC_E_CUDA (-3)    /* a CUDA runtime call failed */
#define QUIC_E_LIMIT (-4)   /* size beyond a documented fixed maximum */
#define QUIC_E_TIMEOUT (-5) /* a bounded wait inside a kernel gave up; results invalid */

const char *quic_last_error(void);
/* Library ABI version; bumped when a struct below changes. */
int quic_abi_version(void);
/* Programmatic dependent launch between the kernels of a decode step is on by
 * default; 0 turns it off process-wide (plain stream order) for A/B timing.
 * No counterpart in the reference, which launches every kernel separately. */
void quic_set_pdl(int enabled);

/* ------------------------------------------------------------------------
 * W4A16 weights.
 *
 * Checkpoint layout (reference src/quant/checkpoint.py:23-36):
 *   weight_packed     int32 [N, K/8]   element k = 8j+i is nibble i of word j
 *   weight_zero_point int32 [N/8, K/G] row n -> word n/8, nibble n%8
 *   weight_scale      fp16  [N, K/G]
 *   w[n,k] = (q - zp[n,k/G]) * scale[n,k/G]
 *
 * Device layout used by the kernels ("W4T", K-major so that a warp reads 32
 * adjacent output columns of one 8-wide k slab with one 128-byte request):
 *   qw int32 [K/8, N], sc fp16 [K/G, N], zp uint8 [K/G, N/2] (two 4-bit zero
 *   points per byte, low nibble = even column).
 * Rows may be permuted on the way (see quic_w4_prepack).  This replaces the
 * Marlin repack of src/quant/marlin.py:105-125.
 * ---------------------------------------------------------------------- */
typedef struct {
  const int32_t *qw; /* [K/8, N] */
  const void *sc;    /* fp16 [K/G, N] */
  const uint8_t *zp; /* [K/G, N/2] */
  const void *bias;  /* fp16 [N] in output-row order of this layout, or NULL */
  int32_t n;
  int32_t k;
  /* Dense form of the same linear (the un-quantised model): fp16 [N, K], K
   * contiguous, rows in the order the packed layout gives its columns; then qw,
   * sc and zp are NULL.  NULL for a packed weight. */
  const void *w16;
} quic_w4_t;

/* Row orders accepted by quic_w4_prepack. */
#define QUIC_ROWS_NATURAL 0
/* Within every block of 64 rows (one attention head) rows are stored as
 * (0,32,1,33,...): the two RoPE partners of a pair become neighbours. */
#define QUIC_ROWS_ROPE_PAIRS 1

/* Repack one checkpoint layer (device pointers) into W4T.  `row_offset` places
 * the layer's N rows at columns [row_offset, row_offset+N) of a fused matrix
 * with `n_total` columns (q|k|v, gate|up).  Replaces
 * src/quant/marlin.py:105 prepack_layer (gptq_repack, marlin_permute_scales,
 * marlin_zero_points). */
int quic_w4_prepack(const int32_t *weight_packed, const void *weight_scale,
                    const int32_t *weight_zero_point, int32_t n, int32_t k,
                    int32_t row_order, int32_t row_offset, int32_t n_total,
                    int32_t *qw, void *sc, uint8_t *zp, void *stream);

/* Dequantise a W4T matrix to fp16 [N, K] (natural row order only).  Used by
 * the bit-exactness tests of the unpack; mirrors
 * src/quant/checkpoint.py:23 dequantize rounded to fp16. */
int quic_w4_dequant(const quic_w4_t *w, void *out_f16, void *stream);

/* y[M,N] = x[M,K] · dequant(W)^T + bias, fp16 in/out, fp32 accumulate.
 * Replaces marlin.forward (kernels/cuda/marlin.cu:4769 marlin_gemm, reached
 * through src/quant/marlin.py:190 marlin_linear).  One row runs the dequant
 * GEMV; two rows and more run the tcgen05 GEMM when `use_tensor` is non-zero
 * (N and K multiples of 128) and the GEMV in row chunks otherwise.  `workspace` (>= quic_w4a16_workspace_bytes)
 * holds split-K partials; its first 16 KB (arrival counters of the tensor
 * path) must be zero before the first call and are left zero. */
int quic_w4a16_linear(const void *x_f16, const quic_w4_t *w, void *y_f16,
                      int32_t m, int32_t use_tensor, void *workspace,
                      void *stream);
int64_t quic_w4a16_workspace_bytes(int32_t m, int32_t n, int32_t k);
/* Error word of the tensor path: 0, or a non-zero code if a bounded wait inside
 * the tcgen05 kernel gave up since the last call (results are then invalid).
 * The word is taken (exchanged with zero on the device).  Synchronises the
 * device; quic_graph_run_host reads the same word together with the tokens,
 * without a synchronisation of its own, and returns QUIC_E_TIMEOUT when it is
 * set.  No reference counterpart (Marlin's lock spins are unbounded,
 * kernels/cuda/marlin.cu:1467-1476). */
int quic_w4a16_tensor_status(void);
/* Test hook for those bounded waits: the GEMM launches that follow probe at
 * most `spin_limit` times per wait (0: the default, 1 << 22) and never request
 * the packed weight tile of k block `skip_kblock` (128 k each; -1: none), so
 * the waits for it run out, every role of the CTA leaves its loop, the status
 * word is set and the kernel returns with its tensor memory released.  Call
 * with (0, -1) to restore normal operation. */
void quic_w4a16_tensor_test_hook(uint32_t spin_limit, int32_t skip_kblock);

/* Test hook for the streamed decode attention (more than 20 rows), for the launches and graph
 * captures that follow.  1: repeat the tile requests made before the dependency wait, as the
 * kernel does when the step counter moved between request and wait.  2: never request the
 * first tile of a row and probe 20000 times at most, so that the bounded waits run out, the
 * kernel sets the error word read by quic_w4a16_tensor_status (code 5 or 6 in bits 16..,
 * bit 14 set) and returns.  0 restores the normal behaviour.  No reference counterpart. */
void quic_attn_stream_test_hook(int32_t mode);

/* ------------------------------------------------------------------------
 * Stand-alone operators with the reference's per-op signatures.
 * ---------------------------------------------------------------------- */

/* y = x * rsqrt(mean(x^2)+eps) * w over rows of 896; optional residual:
 * when `residual` is non-NULL, x := x + residual first and the sum is written
 * to `sum_out`.  Replaces rmsnorm.forward (kernels/cuda/rmsnorm.cu:100) and the
 * torch residual adds of src/model.py:221,224. */
int quic_rmsnorm(const void *x_f16, const void *residual_f16, const void *w_f16,
                 float eps, void *y_f16, void *sum_out_f16, int32_t rows,
                 void *stream);

/* cos/sin tables fp16 [max_pos, 32].  Replaces rope.init_table
 * (kernels/cuda/rope.cu:125); uses accurate cosf/sinf. */
int quic_rope_table_init(const float *inv_freq32, int32_t max_pos, void *cos_f16,
                         void *sin_f16, void *stream);

/* Rotate-half RoPE on x fp16 [B, H, S, 64]; cos/sin fp16 [S,32] (batch_stride
 * 0) or [B,S,32].  Replaces rope.forward (kernels/cuda/rope.cu:85). */
int quic_rope(const void *x_f16, const void *cos_f16, const void *sin_f16,
              void *y_f16, int32_t b, int32_t h, int32_t s,
              int32_t trig_batch_stride, void *stream);

/* Prefill form of "split heads, rotate, append": qkv fp16 [rows, 1152] is the
 * output of the fused QKV linear (columns in the prepacked order: inside every
 * head, rotation pairs adjacent); row r belongs to KV slot slots[r] at position
 * positions[r].  Writes the rotated queries head-major, q_out fp16
 * [14, rows, 64], and the rotated keys / plain values into the layer's cache
 * planes [n_slots, 2, s_max, 64] at (slot, head, position); a row whose slot
 * is outside 0..n_slots-1 or whose position is outside 0..s_max-1 appends
 * nothing (its query is still written).  All tensors 16-byte aligned.
 * Replaces
 * _heads + rope.forward x2 + DynamicCache.update of the reference's attention
 * (src/model.py:138-160). */
int quic_qkv_rope_append(const void *qkv_f16, const int32_t *slots,
                         const int32_t *positions, const void *cos_f16,
                         const void *sin_f16, int32_t max_pos, void *q_out_f16,
                         void *kcache_f16, void *vcache_f16, int32_t s_max,
                         int32_t n_slots, int32_t rows, void *stream);

/* Causal prefill attention of n_seq sequences in one launch (GQA 14:2,
 * head_dim 64).  q_f16 [14, rows, 64] as written by quic_qkv_rope_append;
 * sequence i owns rows seq_start[i] .. seq_start[i] + seq_len[i] - 1; with
 * seq_off (NULL = zeros) its rows are positions seq_off[i] .. of the sequence (a
 * later chunk of a prompt), and its keys and values are positions
 * 0 .. seq_off[i] + seq_len[i] - 1 of KV slot seq_slot[i] in the
 * layer's cache planes [n_slots, 2, s_max, 64] (no padding is stored, so no pad
 * mask exists); out_f16 [rows, 896] token-major; the rows of a sequence whose
 * slot is outside 0..n_slots-1 are left unwritten.  Replaces the reference's
 * prefill attention (kernels/flash_attn_prefill_pytorch.py:10 = torch SDPA with
 * a causal + left-pad mask; kernels/cuda/flash_attn_prefill.cu:87). */
int quic_attn_prefill(const void *q_f16, const void *kcache_f16,
                      const void *vcache_f16, const int32_t *seq_start,
                      const int32_t *seq_len, const int32_t *seq_slot,
                      const int32_t *seq_off, int32_t n_seq, int32_t max_len,
                      int32_t rows,
                      int32_t s_max, int32_t n_slots, float scale,
                      void *out_f16, void *stream);

/* Prompts of 128 tokens and more run quic_attn_prefill on tcgen05 with
 * TMA-staged tiles; shorter ones, and every call after
 * quic_set_prefill_tensor_attention(0), on the mma.sync kernels (for A/B timing
 * and tests). */
void quic_set_prefill_tensor_attention(int enabled);

/* y = silu(gate) * up, rows of 4864.  Replaces swiglu.forward
 * (kernels/cuda/swiglu.cu:37). */
int quic_swiglu(const void *gate_f16, const void *up_f16, void *y_f16,
                int32_t rows, void *stream);
/* The same on the output of the fused gate|up linear, gu [rows, 9728]:
 * y = silu(gu[:, :4864]) * gu[:, 4864:].  The reference runs gate and up as
 * two linears and hands both to swiglu.forward (src/model.py:96-105); here
 * they are one linear, and this form saves slicing its output. */
int quic_swiglu_fused(const void *gu_f16, void *y_f16, int32_t rows,
                      void *stream);

/* Row argmax of fp16 logits [B, V] -> int64 [B]; ties -> lowest index.
 * Replaces sampler.forward (kernels/cuda/sampler.cu:52). */
int quic_argmax(const void *logits_f16, int32_t b, int32_t v, int64_t *out,
                void *stream);

/* y[M,N] = x[M,K] · w[N,K]^T (+ bias), fp16, fp32 accumulate; K multiple of 8.
 * Replaces gemm.forward (kernels/cuda/gemm.cu:36, cuBLAS) for the GEMV-shaped
 * uses on this path (the tied lm_head). */
int quic_gemm_f16(const void *x_f16, const void *w_f16, const void *bias_f16,
                  void *y_f16, int32_t m, int32_t n, int32_t k, void *stream);

/* Tied lm_head fused with (optional) final RMSNorm and greedy argmax:
 * logits[b,:] = norm(x[b,:]) · embed^T, out[b] = argmax (ties -> lowest index, on
 * the fp16-rounded logits).  Replaces, as one kernel, the final norm
 * (src/model.py:298), the cuBLAS lm_head (src/model.py:301 -> kernels/cuda/gemm.cu:36)
 * and torch.argmax (src/engine.py:104).  x fp16 [B,896]; norm_w fp16 [896] or NULL
 * (x already normalised); embed fp16 [vocab,896], vocab even; logits fp16
 * [B,vocab] or NULL; out int64 [B] or NULL; scratch >=
 * quic_lm_head_scratch_bytes(b, vocab) bytes whose first 256 bytes are zero
 * before the first call (the kernel leaves them zero). */
int quic_lm_head_argmax(const void *x_f16, const void *norm_w_f16, float eps,
                        const void *embed_f16, int32_t vocab, int32_t b,
                        void *logits_f16, int64_t *out, void *scratch, void *stream);
int64_t quic_lm_head_scratch_bytes(int32_t b, int32_t vocab);

/* Split-K GQA decode attention.  Replaces flash_attn_decode.forward
 * (kernels/cuda/flash_attn_decode.cu:133): q fp16 [B,14,64]; K and V fp16 with
 * explicit element strides (batch, kv head; tokens are 64 contiguous halves
 * apart); row b attends to tokens [start[b], end[b]) (start == NULL -> 0, the
 * left pad; end == NULL -> s_max).  A row with no tokens yields zeros
 * (flash_attn_decode.cu:118-121).  `scratch` holds the split partials and the
 * arrival counters: quic_attn_scratch_bytes(b, splits) bytes, whose first
 * b*2*4 bytes (the counters) must be zero before the first call; the kernel
 * leaves them zero.  `splits` 0 lets the library choose: quic_attn_pick_splits(b,
 * s_max) splits (size the scratch for that count), or, for 21..128 rows of up to
 * 8192 tokens whose K and V are contiguous [b][2][s_max][64] planes, the streamed
 * kernel of the decode step, which uses no scratch. */
int quic_attn_decode(const void *q_f16, const void *k_f16, const void *v_f16,
                     int64_t stride_b, int64_t stride_h, const int32_t *start,
                     const int32_t *end, int32_t s_max, float scale,
                     void *out_f16, int32_t b, int32_t splits, void *scratch,
                     void *stream);
/* Same operation with no memory from the caller and no allocation anywhere:
 * the split partials and counters sit in an 8 MiB array built into the library
 * image (quic_attn_decode_noalloc_max_bytes(); each GPU that loads the library
 * holds it until the process ends).  This entry point has no counterpart in the
 * reference.  It is meant for callers that cannot allocate where they call
 * from: a serving loop that must not hit the device-wide synchronisation of
 * cudaMalloc/cudaFree, a host runtime that gives a plug-in no allocator, or
 * code running under its own memory budget.
 *  - A request whose quic_attn_scratch_bytes(b, splits) exceeds the array is
 *    refused with QUIC_E_LIMIT; pass a smaller `splits` or use quic_attn_decode.
 *  - The first call on a device (with that device current) looks up the
 *    array's device address; make that first call outside any stream capture.
 *  - All calls share the one array, which keeps the previous call's contents:
 *    the counters are cleared on `stream` before each launch, and two calls
 *    whose kernels can overlap on the GPU (different streams) race. */
int quic_attn_decode_noalloc(const void *q_f16, const void *k_f16, const void *v_f16,
                             int64_t stride_b, int64_t stride_h, const int32_t *start,
                             const int32_t *end, int32_t s_max, float scale,
                             void *out_f16, int32_t b, int32_t splits, void *stream);
int64_t quic_attn_decode_noalloc_max_bytes(void);
/* Same operation, same arguments, for up to quic_attn_decode_cta_max_tokens()
 * (4096) cached tokens, with neither scratch nor counters: one CTA of eight
 * warps covers 512 tokens of a (row, KV head) and the CTAs of a (row, KV head)
 * are a thread-block cluster whose partial results meet in the shared memory
 * of its first CTA.  This is the attention of the decode step at 2..16 rows.
 * Longer caches are refused with QUIC_E_LIMIT. */
int quic_attn_decode_cta(const void *q_f16, const void *k_f16, const void *v_f16,
                         int64_t stride_b, int64_t stride_h, const int32_t *start,
                         const int32_t *end, int32_t s_max, float scale,
                         void *out_f16, int32_t b, void *stream);
int32_t quic_attn_decode_cta_max_tokens(void);
int32_t quic_attn_pick_splits(int32_t b, int32_t s_max);
int64_t quic_attn_scratch_bytes(int32_t b, int32_t splits);

/* ------------------------------------------------------------------------
 * The fused decode step (one token for every active row).
 * Replaces Engine.step + QUICForCausalLM.forward with seq_len == 1
 * (src/engine.py:78-107, src/model.py:272-303): embedding gather, 24 decoder
 * layers, final norm, tied lm_head and greedy argmax, with the KV cache
 * appended in place and the token / position state kept on the device.
 * ---------------------------------------------------------------------- */
typedef struct {
  quic_w4_t qkv;     /* 896 -> 1152, rows in QUIC_ROWS_ROPE_PAIRS order, bias */
  quic_w4_t o;       /* 896 -> 896 */
  quic_w4_t gate_up; /* 896 -> 9728 (gate rows then up rows) */
  quic_w4_t down;    /* 4864 -> 896 */
  const void *ln1;   /* fp16 [896] input_layernorm */
  const void *ln2;   /* fp16 [896] post_attention_layernorm */
} quic_layer_t;

typedef struct {
  int32_t n_layers;
  int32_t vocab;
  float eps;
  int32_t max_pos;           /* rows of the RoPE tables */
  const quic_layer_t *layers; /* HOST array of n_layers entries */
  const void *embed;         /* fp16 [vocab, 896], tied lm_head */
  const void *final_norm;    /* fp16 [896] */
  const void *rope_cos;      /* fp16 [max_pos, 32] */
  const void *rope_sin;
} quic_model_t;

typedef struct {
  /* KV cache fp16 [n_layers][2 (K,V)][n_slots][2 kv heads][s_max][64] */
  void *kv;
  int32_t n_slots;
  int32_t s_max;
  /* Per-slot device state. */
  int32_t *tok; /* [n_slots] token to feed next */
  int32_t *pos; /* [n_slots] tokens already cached = position of `tok` */
  /* Batch rows of this step: slot index per row (device, [batch]). */
  const int32_t *rows;
  int32_t batch;
  /* Generated tokens: out_tokens[(*step_counter % ring) * n_slots + slot]. */
  int32_t *out_tokens;
  int32_t ring;
  int32_t *step_counter; /* device int32, incremented once per step */
  /* Optional fp16 [batch, vocab] logits of the step (NULL to skip). */
  void *logits;
  /* Activation / scratch arena, quic_decode_scratch_bytes() bytes, zeroed
   * once by the caller before first use. */
  void *scratch;
  int32_t attn_splits; /* 0 = choose from ctx_hint */
  int32_t ctx_hint;    /* upper bound of pos+1 over the rows for this launch */
} quic_decode_t;

/* ---- fused prefill --------------------------------------------------------
 * Every admitted prompt through the whole model in one call: embedding gather,
 * 24 x (RMSNorm, W4A16 GEMM, quic_qkv_rope_append, quic_attn_prefill, o_proj,
 * residual + RMSNorm, gate_up, SwiGLU, down, residual + RMSNorm), then the tied
 * lm_head + argmax on the last token of every sequence; fills the KV slots and
 * sets tok[slot] = first generated token, pos[slot] = prompt length.  Replaces
 * the prefill branch of the reference's forward and its splice into the batch
 * (src/model.py:164-199, 272-303; src/engine.py:187-222).  Rows are the tokens
 * of all sequences back to back.  All pointers are device pointers. */
typedef struct {
  const int32_t *ids;       /* [rows] token ids */
  const int32_t *row_slot;  /* [rows] KV slot of the row's sequence */
  const int32_t *row_pos;   /* [rows] position of the row inside its sequence */
  const int32_t *seq_start; /* [n_seq] first row of the sequence */
  const int32_t *seq_len;   /* [n_seq] */
  const int32_t *seq_slot;  /* [n_seq] */
  int32_t rows;
  int32_t n_seq;
  int32_t max_len; /* longest sequence */
  void *kv;        /* cache as in quic_decode_t */
  int32_t n_slots;
  int32_t s_max;
  int32_t *tok; /* [n_slots] */
  int32_t *pos; /* [n_slots] */
  int64_t *first_tokens; /* [n_seq] out */
  void *logits;          /* optional fp16 [n_seq, vocab] of the last positions */
  void *scratch;         /* quic_prefill_scratch_bytes() bytes, zeroed once by the caller */
  /* Chunked prefill: tokens of the sequence already in its slot, [n_seq] or
   * NULL (none).  The rows of the call are then the NEXT tokens of the prompt:
   * row_pos continues from seq_off, attention sees the cached tokens too, and
   * pos[slot] becomes seq_off + seq_len. */
  const int32_t *seq_off;
} quic_prefill_t;
int64_t quic_prefill_scratch_bytes(int32_t rows, int32_t n_seq, int32_t vocab);
int quic_prefill(const quic_model_t *m, const quic_prefill_t *p, void *stream);

/* Which of the three forms of the decode step a batch takes.  Batches of at
 * least quic_set_tensor_min_batch rows (default 16, range 2..17) run every
 * linear on the tcgen05 GEMM and the tensor lm_head; below that, batches of at
 * least quic_set_mma_chain_min_batch rows (default 3, range 2..17) run the
 * five-kernel layer chain with the rows on the M side of mma.sync, whose cost
 * hardly grows with the row count; smaller batches (one row, and two by
 * default) run the GEMV chain.  The defaults are the crossovers measured on
 * B200.  Set them before graphs are captured.  No reference counterpart
 * (Marlin picks its tile shapes per call, kernels/cuda/marlin.cu:3795-3805). */
void quic_set_tensor_min_batch(int32_t batch);
void quic_set_mma_chain_min_batch(int32_t batch);
/* Attention split count the decode step uses for `batch` rows whose contexts are
 * at most `ctx` tokens (pass the result as attn_splits and to the scratch size). */
int32_t quic_decode_pick_splits(int32_t batch, int32_t ctx);
int64_t quic_decode_scratch_bytes(int32_t batch, int32_t vocab, int32_t attn_splits);
/* Number of kernels one quic_decode_step launches. */
int32_t quic_decode_launch_count(const quic_model_t *m, const quic_decode_t *d);
/* Launch one step (kernels chained with programmatic dependent launch). */
int quic_decode_step(const quic_model_t *m, const quic_decode_t *d, void *stream);

/* Capture `steps` consecutive decode steps into a CUDA graph owned by the
 * library; replay with quic_graph_launch.  The same graph stays valid while
 * the pointers in `d`, the batch size and the split count are unchanged:
 * tokens, positions and the row->slot map are read from device memory. */
int quic_decode_graph_create(const quic_model_t *m, const quic_decode_t *d,
                             int32_t steps, void *stream, void **graph_out);
int quic_graph_launch(void *graph, void *stream);
/* One host-driven call of a captured graph, the form the reference's token loop
 * has (src/engine.py:82-84 builds the next-token tensor on the host and copies
 * it to the device, src/engine.py:98-104 synchronises and reads the sampled ids
 * back with .tolist()): copies n_in int32 from host_in to dev_in (skipped when
 * n_in == 0), launches the graph, copies n_out int32 from dev_out to host_out
 * and waits for the stream.  Host buffers should be page-locked. */
int quic_graph_run_host(void *graph, void *stream, const int32_t *host_in,
                        int32_t *dev_in, int32_t n_in, const int32_t *dev_out,
                        int32_t *host_out, int32_t n_out);
int quic_graph_destroy(void *graph);

/* ------------------------------------------------------------------------
 * The decode token loop as one persistent kernel (1..quic_persist_max_rows()
 * batch rows, contexts up to 16 x 256 tokens).  Opt-in: on B200 it measures
 * slower than quic_decode_step's kernel chain (587 vs 352 us per token).
 *
 * Replaces the same reference code as quic_decode_step, for `steps` consecutive
 * greedy tokens in ONE launch: Engine.step + QUICForCausalLM.forward with
 * seq_len == 1 (src/engine.py:78-107, src/model.py:211-224, 272-303).  148
 * resident CTAs walk layers and tokens; a layer phase hands its result to the
 * next through 8-byte {payload, tag} words in `sync`, and the weights stream
 * from a per-CTA copy of the W4 matrices ("W4S", built once by
 * quic_persist_pack from the W4T matrices of quic_model_t) into a
 * shared-memory ring.  Arithmetic and rounding points are those of
 * quic_decode_step.  The kernel is launched cooperatively: it needs a GPU with
 * at least 148 SMs on which all its CTAs can be resident, and it occupies the
 * whole GPU until the burst ends (work on other streams waits).
 *
 *  - `wstream`: quic_persist_stream_bytes(n_layers) bytes, 256-byte aligned,
 *    filled by quic_persist_pack (replaces, like quic_w4_prepack, the repack of
 *    src/quant/marlin.py:105-125).
 *  - `sync`: quic_persist_sync_bytes() bytes, 256-byte aligned, zeroed once by
 *    the caller; one area serves every launch on a stream, launches that can
 *    overlap on the GPU need an area each.
 *  - quic_decode_t: `scratch` is not used; `attn_splits` 0 lets the library
 *    choose from `ctx_hint` (an upper bound of pos + steps over the rows);
 *    `logits` only with steps == 1.
 *  - Every wait inside the kernel is bounded.  If one gives up the kernel ends
 *    early, the tokens of that launch are invalid and the status word of `sync`
 *    is non-zero: quic_decode_persist_status() returns and clears it (it
 *    synchronises the stream), quic_decode_persist_run_host() checks it itself
 *    and returns QUIC_E_TIMEOUT.  No reference counterpart (its kernels have no
 *    bounded waits, kernels/cuda/marlin.cu:1467-1476).
 * ---------------------------------------------------------------------- */
int32_t quic_persist_max_rows(void);
int64_t quic_persist_stream_bytes(int32_t n_layers);
int64_t quic_persist_sync_bytes(void);
/* Attention splits per (row, kv head) for contexts up to `ctx`; more than 16
 * means the context is too long for this kernel (use quic_decode_step). */
int32_t quic_persist_pick_splits(int32_t batch, int32_t ctx);
int quic_persist_pack(const quic_model_t *m, void *wstream_out, void *stream);
int quic_decode_persist(const quic_model_t *m, const quic_decode_t *d,
                        const void *wstream, void *sync, int32_t steps,
                        void *stream);
int quic_decode_persist_status(void *sync, void *stream, int32_t *status_out);
/* The host-driven form (compare quic_graph_run_host; src/engine.py:82-84,
 * 98-104): n_in int32 host -> device, the launch, n_out int32 and the status
 * word device -> host (host_status: one page-locked int32), stream
 * synchronised. */
int quic_decode_persist_run_host(const quic_model_t *m, const quic_decode_t *d,
                                 const void *wstream, void *sync, int32_t steps,
                                 void *stream, const int32_t *host_in,
                                 int32_t *dev_in, int32_t n_in,
                                 const int32_t *dev_out, int32_t *host_out,
                                 int32_t n_out, int32_t *host_status);

#ifdef __cplusplus
}
#endif
#endif /* QUIC_B200_H */
