// Fused prefill: every admitted prompt through the whole model in one library call (no host
// framework ops between the kernels).  It chains the stand-alone entry points of this
// library -- W4A16 linear, RMSNorm (+ residual), quic_qkv_rope_append, quic_attn_prefill,
// quic_swiglu_fused, tied lm_head + argmax -- over activations in a caller-provided scratch
// arena, plus three small kernels of its own (embedding gather, last-row gather, slot state).
#include "decode_kernels.cuh"

namespace quic {
namespace {

constexpr int kPrefillChunk = 8192;  // rows per linear call (bounds the split-K workspace)
constexpr int kGuChunk = 1024;      // rows of gate|up output held at once by the dense fp16 path

inline int64_t align256(int64_t v) { return (v + 255) / 256 * 256; }

struct PrefillArena {
  int64_t lm, h, xn, tmp, qkv, q, attn, gu, act, xlast, ws, total;
};

int64_t linear_ws(int rows) {
  const int m = rows < kPrefillChunk ? rows : kPrefillChunk;
  int64_t w = quic_w4a16_workspace_bytes(m, kQkvN, kHidden);
  const int64_t o = quic_w4a16_workspace_bytes(m, kHidden, kHidden);
  const int64_t g = quic_w4a16_workspace_bytes(m, 2 * kInter, kHidden);
  const int64_t d = quic_w4a16_workspace_bytes(m, kHidden, kInter);
  w = w > o ? w : o;
  w = w > g ? w : g;
  return w > d ? w : d;
}

// The lm_head scratch (whose arrival counter must start zeroed) comes first.
PrefillArena carve_prefill(int rows, int n_seq, int vocab) {
  PrefillArena a;
  int64_t off = 0;
  a.lm = off;
  off += align256(quic_lm_head_scratch_bytes(n_seq, vocab));
  a.h = off;
  off += align256((int64_t)rows * kHidden * 2);
  a.xn = off;
  off += align256((int64_t)rows * kHidden * 2);
  a.tmp = off;
  off += align256((int64_t)rows * kHidden * 2);
  a.qkv = off;
  off += align256((int64_t)rows * kQkvN * 2);
  a.q = off;
  off += align256((int64_t)rows * kHidden * 2);
  a.attn = off;
  off += align256((int64_t)rows * kHidden * 2);
  a.gu = off;
  // gate|up is materialised by the one-row fallback and, kGuChunk rows at a time, by the dense fp16 path
  off += align256((int64_t)(rows < kGuChunk ? rows : kGuChunk) * 2 * kInter * 2);
  a.act = off;
  off += align256((int64_t)rows * kInter * 2);
  a.xlast = off;
  off += align256((int64_t)n_seq * kHidden * 2);
  a.ws = off;
  off += align256(linear_ws(rows));
  a.total = off;
  return a;
}

// x[r] = embed[ids[r]] (ids clamped into the table), 224 threads x 8 bytes per row.
__global__ void __launch_bounds__(224) embed_tokens_kernel(const half* __restrict__ embed,
                                                           const int32_t* __restrict__ ids, int vocab,
                                                           half* __restrict__ x) {
  const int r = blockIdx.x, t = threadIdx.x;
  int id = ids[r];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  reinterpret_cast<uint2*>(x + (size_t)r * kHidden)[t] =
      reinterpret_cast<const uint2*>(embed + (size_t)id * kHidden)[t];
}

// y[i] = x[seq_start[i] + seq_len[i] - 1]: the last position of every sequence.
__global__ void __launch_bounds__(224) gather_last_kernel(const half* __restrict__ x,
                                                          const int32_t* __restrict__ seq_start,
                                                          const int32_t* __restrict__ seq_len,
                                                          half* __restrict__ y) {
  const int i = blockIdx.x, t = threadIdx.x;
  const int r = seq_start[i] + seq_len[i] - 1;
  reinterpret_cast<uint2*>(y + (size_t)i * kHidden)[t] = reinterpret_cast<const uint2*>(x + (size_t)r * kHidden)[t];
}

// tok[slot] = first generated token, pos[slot] = prompt length.
__global__ void set_slot_state_kernel(const int64_t* __restrict__ first, const int32_t* __restrict__ seq_len,
                                      const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_off,
                                      int n_seq, int n_slots, int32_t* __restrict__ tok, int32_t* __restrict__ pos) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_seq) return;
  const int slot = seq_slot[i];
  if (slot < 0 || slot >= n_slots) return;
  tok[slot] = (int32_t)first[i];
  pos[slot] = seq_len[i] + (seq_off != nullptr ? seq_off[i] : 0);
}

// Rows per call of a linear: packed weights beyond kPrefillChunk rows never split K (their CTAs
// fill the SMs many times over), so they need no workspace and one launch covers all rows --
// fewer partial waves than a launch per 8192 rows.  Dense weights keep the chunks.
int linear_chunk(const quic_w4_t& w, int rows) {
  constexpr int kMaxRowsPerLaunch = 1 << 22;  // grid.z = rows / 256 stays far below 65535
  if (w.w16 != nullptr || rows <= kPrefillChunk) return kPrefillChunk;
  return rows < kMaxRowsPerLaunch ? rows : kMaxRowsPerLaunch;
}

// One W4A16 linear over all rows, in chunks that bound the split-K workspace.
int linear_rows(const half* x, const quic_w4_t& w, half* y, int rows, void* ws, void* stream) {
  const int chunk = linear_chunk(w, rows);
  for (int r0 = 0; r0 < rows; r0 += chunk) {
    const int m = rows - r0 < chunk ? rows - r0 : chunk;
    const int rc = quic_w4a16_linear(x + (size_t)r0 * w.k, &w, y + (size_t)r0 * w.n, m, 1, ws, stream);
    if (rc != QUIC_OK) return rc;
  }
  return QUIC_OK;
}

}  // namespace
}  // namespace quic

using namespace quic;

extern "C" int64_t quic_prefill_scratch_bytes(int32_t rows, int32_t n_seq, int32_t vocab) {
  if (rows < 1 || n_seq < 1 || vocab < 2) return 0;
  return carve_prefill(rows, n_seq, vocab).total;
}

extern "C" int quic_prefill(const quic_model_t* m, const quic_prefill_t* p, void* stream) {
  QUIC_REQUIRE(m && p && m->layers && m->embed && m->final_norm && m->rope_cos && m->rope_sin, QUIC_E_ARG,
               "prefill: null model");
  QUIC_REQUIRE(p->ids && p->row_slot && p->row_pos && p->seq_start && p->seq_len && p->seq_slot && p->kv && p->tok &&
                   p->pos && p->first_tokens && p->scratch,
               QUIC_E_ARG, "prefill: null tensor");
  QUIC_REQUIRE(p->rows >= 1 && p->n_seq >= 1 && p->n_seq <= p->rows && p->n_seq <= 65535 && p->max_len >= 1 &&
                   p->max_len <= p->s_max && p->max_len <= m->max_pos && p->n_slots >= 1,
               QUIC_E_SHAPE, "prefill: bad row / sequence counts or a prompt longer than a KV slot");
  cudaStream_t st = (cudaStream_t)stream;
  const int rows = p->rows;
  const PrefillArena ar = carve_prefill(rows, p->n_seq, m->vocab);
  char* base = static_cast<char*>(p->scratch);
  half* h = reinterpret_cast<half*>(base + ar.h);       // residual stream
  half* xn = reinterpret_cast<half*>(base + ar.xn);     // normalised input of the next linear
  half* tmp = reinterpret_cast<half*>(base + ar.tmp);   // o_proj / down output
  half* qkv = reinterpret_cast<half*>(base + ar.qkv);
  half* q = reinterpret_cast<half*>(base + ar.q);
  half* attn = reinterpret_cast<half*>(base + ar.attn);
  half* gu = reinterpret_cast<half*>(base + ar.gu);
  half* act = reinterpret_cast<half*>(base + ar.act);
  half* xlast = reinterpret_cast<half*>(base + ar.xlast);
  void* ws = base + ar.ws;
  const size_t slot_stride = (size_t)kKvHeads * p->s_max * kHeadDim;
  const size_t kv_plane = (size_t)p->n_slots * slot_stride;

  embed_tokens_kernel<<<rows, 224, 0, st>>>((const half*)m->embed, p->ids, m->vocab, h);
  QUIC_CUDA(cudaGetLastError());
  // From here on the kernels are chained with programmatic dependent launch: each one does
  // its set-up (and the GEMMs request their weight tiles) while its predecessor drains.
  QUIC_CUDA(launch_rmsnorm(h, nullptr, (const half*)m->layers[0].ln1, m->eps, xn, nullptr, rows, st));
  int rc = QUIC_OK;
  for (int l = 0; l < m->n_layers; ++l) {
    const quic_layer_t& L = m->layers[l];
    half* kc = static_cast<half*>(p->kv) + (size_t)(2 * l) * kv_plane;
    half* vc = kc + kv_plane;
    if ((rc = linear_rows(xn, L.qkv, qkv, rows, ws, stream)) != QUIC_OK) return rc;
    QUIC_CUDA(launch_qkv_rope_append(qkv, p->row_slot, p->row_pos, (const half*)m->rope_cos, (const half*)m->rope_sin,
                                     m->max_pos, q, kc, vc, p->s_max, p->n_slots, rows, st, true));
    if ((rc = attn_prefill_launch(q, kc, vc, p->seq_start, p->seq_len, p->seq_slot, p->seq_off, p->n_seq, p->max_len,
                                  rows, p->s_max, p->n_slots, 0.125f /* 64^-0.5, src/model.py:129 */, attn, st, true)) != QUIC_OK)
      return rc;
    if ((rc = linear_rows(attn, L.o, tmp, rows, ws, stream)) != QUIC_OK) return rc;
    // h += o ; xn = norm(h)
    QUIC_CUDA(launch_rmsnorm(tmp, h, (const half*)L.ln2, m->eps, xn, h, rows, st));
    if (L.gate_up.w16 != nullptr) {  // dense fp16 weights: GEMM, then SwiGLU, a chunk of rows at a time
      for (int r0 = 0; r0 < rows; r0 += kGuChunk) {
        const int mrows = rows - r0 < kGuChunk ? rows - r0 : kGuChunk;
        if ((rc = linear_rows(xn + (size_t)r0 * kHidden, L.gate_up, gu, mrows, ws, stream)) != QUIC_OK) return rc;
        QUIC_CUDA(launch_swiglu_fused(gu, act + (size_t)r0 * kInter, mrows, st));
      }
    } else if (rows >= 2) {  // gate|up GEMM with SwiGLU in its epilogue: the [rows, 9728] intermediate never exists
      const int chunk = linear_chunk(L.gate_up, rows);
      for (int r0 = 0; r0 < rows; r0 += chunk) {
        const int mrows = rows - r0 < chunk ? rows - r0 : chunk;
        if ((rc = w4a16_gemm_tc_swiglu(xn + (size_t)r0 * kHidden, L.gate_up, act + (size_t)r0 * kInter, mrows, st)) !=
            QUIC_OK)
          return rc;
      }
    } else {
      if ((rc = linear_rows(xn, L.gate_up, gu, rows, ws, stream)) != QUIC_OK) return rc;
      QUIC_CUDA(launch_swiglu_fused(gu, act, rows, st));
    }
    if ((rc = linear_rows(act, L.down, tmp, rows, ws, stream)) != QUIC_OK) return rc;
    const void* next_ln = (l + 1 < m->n_layers) ? m->layers[l + 1].ln1 : m->final_norm;
    QUIC_CUDA(launch_rmsnorm(tmp, h, (const half*)next_ln, m->eps, xn, h, rows, st));
  }
  // xn holds the finally normalised rows: lm_head + argmax on the last one of every sequence
  gather_last_kernel<<<p->n_seq, 224, 0, st>>>(xn, p->seq_start, p->seq_len, xlast);
  QUIC_CUDA(cudaGetLastError());
  if ((rc = quic_lm_head_argmax(xlast, nullptr, m->eps, m->embed, m->vocab, p->n_seq, p->logits, p->first_tokens,
                                base + ar.lm, stream)) != QUIC_OK)
    return rc;
  set_slot_state_kernel<<<(p->n_seq + 127) / 128, 128, 0, st>>>(p->first_tokens, p->seq_len, p->seq_slot, p->seq_off,
                                                               p->n_seq, p->n_slots, p->tok, p->pos);
  QUIC_CUDA(cudaGetLastError());
  return QUIC_OK;
}
