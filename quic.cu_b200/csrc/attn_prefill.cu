// Causal prefill attention over KV slots (GQA 14:2, head_dim 64), all admitted sequences in
// one launch.  Queries come head-major from quic_qkv_rope_append, keys and values are read
// from the slots that kernel has just filled, and the output is written token-major
// [rows, 896], which is the layout the o_proj GEMM consumes.
//
// Flash-attention-2 style on mma.sync.m16n8k16: a CTA owns 16 consecutive query rows of one
// head; its four warps walk alternate tiles of 32 keys up to the causal bound, each with an
// online softmax, and their states are merged through shared memory at the end.
// The fragment mappings are those of attn_warp.cuh (K fragments are the lane's own 32
// contiguous bytes of a key row, probabilities go from the score fragments straight into the
// A operand of p.V, V pairs are built with byte permutes); the difference to decode is that
// all 16 rows of the M tile are real queries, so every lane carries two rows (g and g + 8).
// No shared memory: K/V tiles are re-read through L1 / L2 by the warps that need them.
#include "attn_warp.cuh"
#include "decode_kernels.cuh"

namespace quic {
namespace {

// Read-only load that allocates in L1: the warps of a CTA walk the same K/V tiles at
// about the same time, so repeated reads of a tile are L1 hits.  (The cache rows were
// written by an earlier kernel; L1 holds nothing stale at kernel start.)
__device__ __forceinline__ uint4 ldg_l1_u128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Two forms.  kSplitKeys: the 4 warps of a CTA share 16 query rows and take alternate key
// tiles (the walk over a row's keys is a serial chain per warp -- load, q.K, softmax, p.V per
// tile -- and four warps cut it to a quarter; their states are merged through shared memory):
// for launches with few rows, which are bound by that chain (one sequence of 512 tokens: 20 ->
// 10 us).  Otherwise 2 warps per CTA own 16 query rows each and share their K/V tiles through
// L1: for launches with many rows, which are bound by cache traffic (16 x 512: 72 us against 85).
constexpr int kPfSplitWarps = 4;
constexpr int kPfRowWarps = 2;
constexpr int kGroupHeads = kHeads / kKvHeads;

struct PrefillAttnArgs {
  const half* q;        // [14][rows][64]
  const half* kcache;   // [n_slots][2][s_max][64]
  const half* vcache;
  const int32_t* seq_start;  // [n_seq] first row of the sequence in q / out
  const int32_t* seq_len;    // [n_seq]
  const int32_t* seq_slot;   // [n_seq]
  const int32_t* seq_off;    // [n_seq] tokens of the sequence already in its slot (a later chunk of a prompt), or nullptr
  half* out;            // [rows][896]
  int32_t rows;
  int32_t s_max;
  int32_t n_slots;
  float scale;
};

template <bool kSplitKeys>
__global__ void __launch_bounds__((kSplitKeys ? kPfSplitWarps : kPfRowWarps) * 32)
    attn_prefill_kernel(const PrefillAttnArgs a) {
  constexpr int kPfWarps = kSplitKeys ? kPfSplitWarps : kPfRowWarps;
  constexpr int kPfRows = kSplitKeys ? 16 : 16 * kPfRowWarps;  // query rows per CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int head = blockIdx.y, seq = blockIdx.z;
  pdl_trigger_early();
  pdl_wait();  // queries and cache rows come from the kernels before this one
  const int len = a.seq_len[seq];
  // the longest key ranges first: CTAs of late query rows are launched before the short ones
  const int r0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * kPfRows + (kSplitKeys ? 0 : warp * 16);  // first query row of the warp
  if (r0 >= len) return;
  const int start = a.seq_start[seq];
  const int off = a.seq_off != nullptr ? max(a.seq_off[seq], 0) : 0;  // query row r sits at position off + r
  const int kv_len = off + len;
  const int slot = a.seq_slot[seq];
  if (slot < 0 || slot >= a.n_slots) return;  // no such slot: the sequence's rows stay unwritten
  const int kvh = head / kGroupHeads;
  const half* kbase = a.kcache + ((size_t)slot * kKvHeads + kvh) * a.s_max * kHeadDim;
  const half* vbase = a.vcache + ((size_t)slot * kKvHeads + kvh) * a.s_max * kHeadDim;
  const int last_tok = kv_len - 1, last_row = len - 1;

  // Q fragments of rows r0 + g (a0, a2) and r0 + g + 8 (a1, a3): dims 16c + 4ks + {0,1} | {2,3}
  uint32_t qa[4][4];
  {
    const int ra = min(r0 + g, last_row), rb = min(r0 + g + 8, last_row);  // rows past the end mirror the last
    const half* qa_p = a.q + ((size_t)head * a.rows + start + ra) * kHeadDim + 16 * c;
    const half* qb_p = a.q + ((size_t)head * a.rows + start + rb) * kHeadDim + 16 * c;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const uint2 ua = *reinterpret_cast<const uint2*>(qa_p + 4 * ks);
      const uint2 ub = *reinterpret_cast<const uint2*>(qb_p + 4 * ks);
      qa[ks][0] = ua.x;
      qa[ks][1] = ub.x;
      qa[ks][2] = ua.y;
      qa[ks][3] = ub.y;
    }
  }
  const int pos_a = off + r0 + g, pos_b = off + r0 + g + 8;  // causal bounds of the lane's two rows
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

  const int t_stop = min(off + r0 + 16, kv_len);  // keys 0 .. t_stop - 1 are visible to some row of the warp
  // Warp w takes the key tiles w, w + 4, ...: the walk over a row's keys is a serial chain per
  // warp (load, q.K, softmax, p.V per tile), and four warps cut it to a quarter.
  for (int t0 = kSplitKeys ? 32 * warp : 0; t0 < t_stop; t0 += kSplitKeys ? 32 * kPfWarps : 32) {
    // ---- loads: K rows t0 + 8nb + g, bytes [32c, 32c+32); V rows t0 + 16j + 2c + {0,1,8,9}, dims 8g..8g+7
    uint4 kr[4][2], vr[2][4];
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
      const uint4* kp = reinterpret_cast<const uint4*>(kbase + (size_t)min(t0 + 8 * nb + g, last_tok) * kHeadDim + 16 * c);
      kr[nb][0] = ldg_l1_u128(kp);
      kr[nb][1] = ldg_l1_u128(kp + 1);
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int tb = t0 + 16 * j + 2 * c;
      vr[j][0] = ldg_l1_u128(vbase + (size_t)min(tb, last_tok) * kHeadDim + 8 * g);
      vr[j][1] = ldg_l1_u128(vbase + (size_t)min(tb + 1, last_tok) * kHeadDim + 8 * g);
      vr[j][2] = ldg_l1_u128(vbase + (size_t)min(tb + 8, last_tok) * kHeadDim + 8 * g);
      vr[j][3] = ldg_l1_u128(vbase + (size_t)min(tb + 9, last_tok) * kHeadDim + 8 * g);
    }
    // ---- scores: d[nb][0..1] row g, d[nb][2..3] row g + 8, tokens t0 + 8nb + 2c + {0,1}
    float d[4][4];
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) d[nb][0] = d[nb][1] = d[nb][2] = d[nb][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {  // k steps outermost: consecutive mma are independent
#pragma unroll
      for (int nb = 0; nb < 4; ++nb) {
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&kr[nb][0]);
        mma16816(d[nb], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], u[2 * ks], u[2 * ks + 1]);
      }
    }
    float mt[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int t = t0 + 8 * nb + 2 * c + e;
        d[nb][e] = (t <= pos_a && t < kv_len) ? d[nb][e] * a.scale : -INFINITY;
        d[nb][2 + e] = (t <= pos_b && t < kv_len) ? d[nb][2 + e] * a.scale : -INFINITY;
        mt[0] = fmaxf(mt[0], d[nb][e]);
        mt[1] = fmaxf(mt[1], d[nb][2 + e]);
      }
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mt[r] = fmaxf(mt[r], __shfl_xor_sync(0xffffffffu, mt[r], 1));
      mt[r] = fmaxf(mt[r], __shfl_xor_sync(0xffffffffu, mt[r], 2));
      const float m_new = fmaxf(m_run[r], mt[r]);
      alpha[r] = (m_run[r] == -INFINITY) ? 0.f : __expf(m_run[r] - m_new);  // m_new finite whenever m_run is
      m_run[r] = m_new;
    }
    uint32_t pa[2][4];  // P as A fragments per 16-token k step: a0 (row g), a1 (row g+8), a2, a3 (second 8 tokens)
    float l_add[2] = {0.f, 0.f};
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float s0 = d[nb][2 * r], s1 = d[nb][2 * r + 1];
        const float p0 = (s0 == -INFINITY) ? 0.f : __expf(s0 - m_run[r]);
        const float p1 = (s1 == -INFINITY) ? 0.f : __expf(s1 - m_run[r]);
        const half2 ph = __floats2half2_rn(p0, p1);
        l_add[r] += __low2float(ph) + __high2float(ph);  // the sum uses the rounded probabilities that multiply V
        pa[nb >> 1][2 * (nb & 1) + r] = *reinterpret_cast<const uint32_t*>(&ph);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * alpha[r] + l_add[r];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o[j][0] *= alpha[0];
      o[j][1] *= alpha[0];
      o[j][2] *= alpha[1];
      o[j][3] *= alpha[1];
    }
    // ---- O += P V ; mma j covers dims {8n + j}: lane n = g supplies dim 8g + j
#pragma unroll
    for (int jk = 0; jk < 2; ++jk) {
      const uint32_t* v0 = reinterpret_cast<const uint32_t*>(&vr[jk][0]);  // token 2c
      const uint32_t* v1 = reinterpret_cast<const uint32_t*>(&vr[jk][1]);  // token 2c + 1
      const uint32_t* v2 = reinterpret_cast<const uint32_t*>(&vr[jk][2]);  // token 2c + 8
      const uint32_t* v3 = reinterpret_cast<const uint32_t*>(&vr[jk][3]);  // token 2c + 9
#pragma unroll
      for (int w = 0; w < 4; ++w) {  // word w holds dims 8g + 2w, 8g + 2w + 1
        const uint32_t b0_lo = __byte_perm(v0[w], v1[w], 0x5410), b0_hi = __byte_perm(v0[w], v1[w], 0x7632);
        const uint32_t b1_lo = __byte_perm(v2[w], v3[w], 0x5410), b1_hi = __byte_perm(v2[w], v3[w], 0x7632);
        mma16816(o[2 * w], pa[jk][0], pa[jk][1], pa[jk][2], pa[jk][3], b0_lo, b1_lo);
        mma16816(o[2 * w + 1], pa[jk][0], pa[jk][1], pa[jk][2], pa[jk][3], b0_hi, b1_hi);
      }
    }
  }

  // ---- (split keys) merge the warps' partial softmax states through shared memory, warp 0 finishes
  constexpr int kSm = kSplitKeys ? kPfSplitWarps : 1;
  __shared__ float sm_m[kSm][16], sm_l[kSm][16];
  __shared__ float sm_o[kSm][32][32 + 1];  // [warp][value index][lane], padded
  const int sw = kSplitKeys ? warp : 0;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    l_run[r] = l;
    if (kSplitKeys && c == 0) {
      sm_m[sw][g + 8 * r] = m_run[r];
      sm_l[sw][g + 8 * r] = l;
    }
  }
  if (kSplitKeys) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) sm_o[sw][4 * j + e][lane] = o[j][e];
    __syncthreads();
    if (warp != 0) return;
  }
  // C columns 2c, 2c+1 of mma j are dims 16c + j and 16c + 8 + j; rows g (o[j][0..1]) and g + 8 (o[j][2..3])
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int rr = g + 8 * r;
    float wgt[kSm], l = 0.f;
    if (kSplitKeys) {
      float mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < kSm; ++w) mx = fmaxf(mx, sm_m[w][rr]);
#pragma unroll
      for (int w = 0; w < kSm; ++w) {
        wgt[w] = (sm_m[w][rr] == -INFINITY) ? 0.f : __expf(sm_m[w][rr] - mx);
        l += wgt[w] * sm_l[w][rr];
      }
    } else {
      wgt[0] = 1.f;
      l = l_run[r];
    }
    const int row = r0 + rr;
    if (row >= len) continue;
    const float inv = l > 0.f ? 1.f / l : 0.f;
    float v[8][2];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float acc = 0.f;
        if (kSplitKeys) {
#pragma unroll
          for (int w = 0; w < kSm; ++w) acc += wgt[w] * sm_o[w][4 * j + 2 * r + e][lane];
        } else {
          acc = o[j][2 * r + e];
        }
        v[j][e] = acc * inv;
      }
    half* op = a.out + (size_t)(start + row) * kHidden + head * kHeadDim + 16 * c;
    uint4 lo, hi;
    lo.x = pack_half2(v[0][0], v[1][0]);
    lo.y = pack_half2(v[2][0], v[3][0]);
    lo.z = pack_half2(v[4][0], v[5][0]);
    lo.w = pack_half2(v[6][0], v[7][0]);
    hi.x = pack_half2(v[0][1], v[1][1]);
    hi.y = pack_half2(v[2][1], v[3][1]);
    hi.z = pack_half2(v[4][1], v[5][1]);
    hi.w = pack_half2(v[6][1], v[7][1]);
    *reinterpret_cast<uint4*>(op) = lo;
    *reinterpret_cast<uint4*>(op + 8) = hi;
  }
}

}  // namespace
}  // namespace quic

namespace quic {
// Prompts of 128 tokens and more take the tcgen05 kernel (quic_set_prefill_tensor_attention).
bool g_prefill_tc = true;

int attn_prefill_launch(const void* q, const void* kcache, const void* vcache, const int32_t* seq_start,
                        const int32_t* seq_len, const int32_t* seq_slot, const int32_t* seq_off, int32_t n_seq,
                        int32_t max_len, int32_t rows, int32_t s_max, int32_t n_slots, float scale, void* out,
                        cudaStream_t stream, bool pdl) {
  QUIC_REQUIRE(q && kcache && vcache && seq_start && seq_len && seq_slot && out, QUIC_E_ARG,
               "attn_prefill: null tensor");
  QUIC_REQUIRE(n_seq >= 0 && n_seq <= 65535 && rows >= 0 && max_len >= 0 && s_max >= 1 && max_len <= s_max &&
                   n_slots >= 1,
               QUIC_E_SHAPE, "attn_prefill: bad sequence count or lengths");
  QUIC_REQUIRE(((uintptr_t)q % 16 == 0) && ((uintptr_t)kcache % 16 == 0) && ((uintptr_t)vcache % 16 == 0) &&
                   ((uintptr_t)out % 16 == 0),
               QUIC_E_ARG, "attn_prefill: tensors must be 16-byte aligned");
  if (n_seq == 0 || rows == 0 || max_len == 0) return QUIC_OK;
  if (g_prefill_tc && attn_prefill_tc_supported(n_seq, max_len, rows, s_max, n_slots))
    return attn_prefill_tc_launch(q, kcache, vcache, seq_start, seq_len, seq_slot, seq_off, n_seq, max_len, rows,
                                  s_max, n_slots, scale, out, stream, pdl);
  PrefillAttnArgs a = {};
  a.q = (const half*)q;
  a.kcache = (const half*)kcache;
  a.vcache = (const half*)vcache;
  a.seq_start = seq_start;
  a.seq_len = seq_len;
  a.seq_slot = seq_slot;
  a.seq_off = seq_off;
  a.out = (half*)out;
  a.rows = rows;
  a.s_max = s_max;
  a.n_slots = n_slots;
  a.scale = scale > 0.f ? scale : 0.125f;
  if (n_seq == 1 || rows <= 1024) {  // one sequence or few rows: bound by the per-row key walk
    dim3 grid((max_len + 15) / 16, kHeads, n_seq);
    QUIC_CUDA(launch(attn_prefill_kernel<true>, grid, dim3(kPfSplitWarps * 32), 0, stream, pdl, a));
  } else {
    constexpr int kRows = 16 * kPfRowWarps;
    dim3 grid((max_len + kRows - 1) / kRows, kHeads, n_seq);
    QUIC_CUDA(launch(attn_prefill_kernel<false>, grid, dim3(kPfRowWarps * 32), 0, stream, pdl, a));
  }
  return QUIC_OK;
}
}  // namespace quic

extern "C" int quic_attn_prefill(const void* q, const void* kcache, const void* vcache, const int32_t* seq_start,
                                 const int32_t* seq_len, const int32_t* seq_slot, const int32_t* seq_off,
                                 int32_t n_seq, int32_t max_len, int32_t rows, int32_t s_max, int32_t n_slots,
                                 float scale, void* out, void* stream) {
  return quic::attn_prefill_launch(q, kcache, vcache, seq_start, seq_len, seq_slot, seq_off, n_seq, max_len, rows,
                                   s_max, n_slots, scale, out, (cudaStream_t)stream, false);
}

extern "C" void quic_set_prefill_tensor_attention(int enabled) { quic::g_prefill_tc = enabled != 0; }
