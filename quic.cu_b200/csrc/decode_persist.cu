// The whole decode token loop as ONE persistent kernel: 148 resident CTAs walk the 24 layers
// and the lm_head of every token of a burst and hand each layer phase's result to the next
// through tagged words in L2; the weights stream from HBM into a shared-memory ring that is
// independent of that dependency chain.
//
// Replaces, for up to kPMaxRows batch rows, Engine.step + QUICForCausalLM.forward with
// seq_len == 1 of the reference (src/engine.py:78-107, src/model.py:211-224, 272-303): the same
// arithmetic and fp16 rounding points as the kernel chain of decode_layers.cu / lm_head.cu
// (dequant kernels/cuda/marlin.cu:2290-2313, RMSNorm rmsnorm.cu:39-86, RoPE rope.cu:44-61,
// attention flash_attn_decode.cu:82-130, SwiGLU swiglu.cu:31-33, argmax sampler.cu:38-40).
//
// Why one kernel: a dependent launch costs 0.7 us on this part even for an empty kernel and a
// token has 121 of them, each followed by a round trip to L2 for its input vector.  Here a
// phase ends with 8-byte stores {payload, tag} and the next phase polls exactly the words it
// needs, so the data and the "ready" signal travel together.
//
// Work split (CTA c of 148, 8 warps).  The unit of a linear is (output column, quantisation
// group): 128 weights; a thread owns up to two units per phase, eight adjacent lanes share a
// group so their activation loads are one broadcast:
//   qkv      c < 144   8 columns x 7 groups = 56 units
//   attn     tasks (row, kv head, split) dealt round-robin; a warp owns 32 tokens
//   o_proj   c < 112   8 columns x 7 groups; merges the attention splits itself
//   gate|up  all       17 or 16 column pairs of gate and of up x 7 groups = 476 / 448 units
//   down     c < 112   8 columns x 38 groups = 304 units; adds the residual
//   lm_head  all       a contiguous range of table rows; candidates exchanged, every CTA
//                      finds the argmax, CTA 0 updates the slot state
// A thread dequantises its units into registers BEFORE the phase's input is polled, so the
// critical path of a phase is poll -> norm -> 128 mixed-precision FMA per unit and row ->
// reduce over the groups in shared memory -> store.
//
// What was measured on the way (B200, 24 layers, one row at 640 tokens of context):
//   * a tagged-word hand-off between 148 resident CTAs costs 1.0-1.2 us (448 words from 112
//     producers), an arrival counter with release/acquire 1.75 us, an empty dependent kernel
//     launch 0.72 us;
//   * mma.sync.m16n8k16 issues once per ~12 cycles per SM partition: with one to four of its
//     sixteen rows in use the plain FMAs are several times cheaper, so the linears use them;
//   * fp16x2 arithmetic issues at half rate, so dequantising a layer's 58 KB of packed weights
//     costs an SM ~1.4 us of issue time: it has to overlap the waits;
//   * almost all of an SM's L1 is carved out as shared memory here, so a register spill is a
//     round trip to L2; 16 warps x 128 registers spilled in every phase (33 us per layer),
//     8 warps x 255 registers still spill around the one call left in the layer loop (21 us
//     per layer, 587 us per token against 352 us for the kernel chain).
// The kernel is therefore opt-in (the kernel chain stays the default for one to three rows).
//
// Weight stream ("W4S"): per layer and CTA one contiguous blob, copied by cp.async.bulk into
// a two-layer ring two layers ahead.  A region of U units holds piece j (words 4j..4j+3 of a
// unit's 16 packed words) of unit u at (j * U + u) * 16, then U x {fp16 scale, u16 zero point}.
//
// Waits: every poll and every mbarrier wait is bounded; on a timeout the CTA records a code
// in the status word, the other CTAs see it within a few hundred probes, all wait for their
// own copies in flight and return.  The kernel is launched cooperatively (all CTAs resident).
#include "attn_warp.cuh"
#include "decode_kernels.cuh"
#include "tc_common.cuh"

namespace quic {
namespace {

using u64 = unsigned long long;

constexpr int kPCtas = 148;
constexpr int kPThreads = 256;           // 8 warps: 255 registers per thread, two weight units each
constexpr int kPWarps = kPThreads / 32;
constexpr int kUnitsPerThread = 2;
constexpr int kPMaxRows = 4;
constexpr int kPMaxSplits = 16;
constexpr int kPMaxLayers = 30;

constexpr int kUnitBytes = 68;          // 16 packed words + {fp16 scale, u16 zero point}
constexpr int kQkvCtas = kQkvN / 8;     // 144
constexpr int kOCtas = kHidden / 8;     // 112
constexpr int kGroupsH = kHidden / kGroup;  // 7
constexpr int kGroupsI = kInter / kGroup;   // 38
constexpr int kUnitsH = 8 * kGroupsH;       // 56 units of a qkv / o_proj CTA
constexpr int kUnitsD = 8 * kGroupsI;       // 304 units of a down CTA
// gate | up: 2432 column pairs over 148 CTAs: the first 64 CTAs own 17 pairs, the others 16
constexpr int kGuBigCtas = 64;
constexpr int kUnitsGuMax = 17 * 4 * kGroupsH;  // 476

constexpr int kOffQkv = 0;
constexpr int kOffBias = kOffQkv + kUnitsH * kUnitBytes;   // 3808
constexpr int kOffO = kOffBias + 16;                        // 3824
constexpr int kOffDown = kOffO + kUnitsH * kUnitBytes;      // 7632
constexpr int kOffGu = kOffDown + kUnitsD * kUnitBytes;     // 28304
constexpr int kBlobBytes = kOffGu + kUnitsGuMax * kUnitBytes;  // 60672
constexpr int kBlobStride = 60928;
static_assert(kBlobBytes <= kBlobStride && kBlobStride % 256 == 0, "blob layout");
static_assert(kOffO % 16 == 0 && kOffDown % 16 == 0 && kOffGu % 16 == 0, "bulk copies need 16-byte pieces");
static_assert(kUnitsGuMax <= kUnitsPerThread * kPThreads, "at most two units per thread");

// words per row of the exchange buffers
constexpr int kXWords = kHidden / 2;              // 448
constexpr int kQkvWords = kQkvN / 2;              // 576
constexpr int kAttWords = 7 * 66;                 // per (row, kv head, split): 7 heads x (64 o + m + l)
constexpr int kActWords = kInter / 2;             // 2432

// phase ids inside a tag
constexpr int kTagX = 0, kTagQkv = 1, kTagAtt = 2, kTagXb = 3, kTagAct = 4, kTagCand = 6;

constexpr uint32_t kPollLimit = 1u << 20;

// column pairs of gate (and of up) owned by a CTA, and the first of them
__host__ __device__ __forceinline__ int gu_pairs_of(int cta) { return cta < kGuBigCtas ? 17 : 16; }
__host__ __device__ __forceinline__ int gu_pair0_of(int cta) {
  return cta < kGuBigCtas ? 17 * cta : 17 * kGuBigCtas + 16 * (cta - kGuBigCtas);
}

struct SyncLayout {
  int64_t xa, xb, qkv, att, act, cand, total;  // byte offsets
};
__host__ __device__ inline SyncLayout sync_layout() {
  SyncLayout s;
  int64_t off = 256;
  s.xa = off;   off += (int64_t)8 * kPMaxRows * kXWords;
  s.xb = off;   off += (int64_t)8 * kPMaxRows * kXWords;
  s.qkv = off;  off += (int64_t)8 * kPMaxRows * kQkvWords;
  s.att = off;  off += (int64_t)8 * kPMaxRows * kKvHeads * kPMaxSplits * kAttWords;
  s.act = off;  off += (int64_t)8 * kPMaxRows * kActWords;
  s.cand = off; off += (int64_t)8 * kPCtas * kPMaxRows * 2;
  s.total = (off + 255) / 256 * 256;
  return s;
}

struct PersistArgs {
  const unsigned char* blobs;  // [n_layers][148][kBlobStride]
  const half* lnw;             // [n_layers][2][896]
  const half* embed;
  const half* final_norm;
  const half* cos_t;
  const half* sin_t;
  int32_t n_layers, vocab, max_pos;
  float eps;
  half* kv;
  int32_t n_slots, s_max;
  int32_t* tok;
  int32_t* pos;
  const int32_t* rows;
  int32_t batch;
  int32_t* out_tokens;
  int32_t ring;
  int32_t* step_counter;
  half* logits;
  unsigned char* sync;  // header + exchange buffers
  int32_t steps;
  int32_t splits;  // attention splits per (row, kv head)
  int32_t chunk;   // tokens per split, multiple of 32, <= 448
};

// ---- tagged words -----------------------------------------------------------------------
__device__ __forceinline__ void st_tag(u64* p, uint32_t payload, uint32_t tag) {
  const u64 v = ((u64)tag << 32) | payload;
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_tag_release(u64* p, uint32_t payload, uint32_t tag) {
  const u64 v = ((u64)tag << 32) | payload;
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ u64 ld_tag(const u64* p) {
  u64 v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ u64 ld_tag_acquire(const u64* p) {
  u64 v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t make_tag(uint32_t epoch, int layer, int phase) {
  return (epoch << 8) | (uint32_t)(layer * 8 + phase);
}
__device__ __forceinline__ uint32_t next_epoch(uint32_t e) {
  e = (e + 1) & 0xFFFFFFu;
  return e == 0 ? 1u : e;
}

constexpr int kRedStride = 480;  // >= the most units a CTA has in a phase (476)
// Dynamic shared memory of the kernel; every region sits at a compile-time offset.
extern __shared__ __align__(128) unsigned char smem_base[];

constexpr int kAttnPartBytes = (kPWarps * kAttWords * 4 + 127) / 128 * 128;  // warp partials [15][7][66] fp32
constexpr int scratch_bytes_of(int M) {
  const int act = M * kInter * 2;
  const int attn = kAttnPartBytes + 9 * kHeadDim * 2;  // + q (7 heads), k, v rows of the decoded token
  return ((act > attn ? act : attn) + 255) / 256 * 256;
}
template <int M>
struct SL {  // byte offsets
  static constexpr int ring = 0;                          // 2 x kBlobStride
  static constexpr int xraw = 2 * kBlobStride;            // [M][896] residual stream entering the current norm
  static constexpr int xn = xraw + M * kHidden * 2;       // [M][896] input of the current linear (perm8) / lm_head
  static constexpr int scr = xn + M * kHidden * 2;        // down input [M][4864] (perm8) | attention scratch
  static constexpr int red = scr + scratch_bytes_of(M);   // [M][kRedStride] per-unit partial sums
  static constexpr int ssq = red + M * kRedStride * 4;    // [M][16]
  static constexpr int st = ssq + M * 16 * 4;             // pos[M] slot[M] tok[M], blobs requested, abort flag
  static constexpr int bars = st + 64;                    // two mbarriers
  static constexpr int args = bars + 64;                  // SmArgs
  static constexpr int total = args + 384;
  static_assert(xraw % 128 == 0 && xn % 128 == 0 && scr % 128 == 0 && red % 16 == 0 && ssq % 16 == 0 && bars % 8 == 0,
                "shared-memory regions are read with 16-byte loads");
};
static_assert(kAttnPartBytes % 16 == 0, "the q/k/v rows behind the warp partials are read with 16-byte loads");
#define XRAW (reinterpret_cast<half*>(smem_base + SL<M>::xraw))
#define XN (reinterpret_cast<half*>(smem_base + SL<M>::xn))
#define SCR (smem_base + SL<M>::scr)
#define RED (reinterpret_cast<float*>(smem_base + SL<M>::red))
#define SSQ (reinterpret_cast<float*>(smem_base + SL<M>::ssq))
#define ST (reinterpret_cast<int*>(smem_base + SL<M>::st))
// exchange buffers in global memory (`a` = launch arguments, `sl` = sync_layout() in scope)
#define XA (reinterpret_cast<u64*>(a.sync + sl.xa))
#define XB (reinterpret_cast<u64*>(a.sync + sl.xb))
#define QKVX (reinterpret_cast<u64*>(a.sync + sl.qkv))
#define ATTX (reinterpret_cast<u64*>(a.sync + sl.att))
#define ACTX (reinterpret_cast<u64*>(a.sync + sl.act))
#define CANDX (reinterpret_cast<u64*>(a.sync + sl.cand))

// Launch arguments and the few launch-wide values the phases need, kept in shared memory (each
// phase is a function of its own; see token_kernel).
struct SmArgs {
  PersistArgs a;
  uint32_t poll_limit;
  int32_t withhold_layer;
  int32_t step0;
};
static_assert(sizeof(SmArgs) <= 384, "SmArgs region");

// What a poll needs to know.
struct Ctx {
  uint32_t* status;     // global status word
  uint32_t poll_limit;  // probes before a poll gives up
};

// Polls up to U tagged words (addresses from `addr(u)`, u < n) until each carries `tag`;
// all loads of a round are in flight together.  On a timeout (code recorded in the status
// word) or when another CTA has reported one, sets `bad` and returns zeros for the missing
// words; the caller folds `bad` into its next CTA barrier (__syncthreads_or).
template <int U, typename AddrFn>
__device__ __forceinline__ void poll_words(const Ctx& c, AddrFn addr, int n, uint32_t tag, uint32_t (&val)[U],
                                           bool& bad, bool acquire = false) {
  static_assert(U <= 16, "pending words are tracked in a bit mask");
  // everything lives in registers: a bit per pending word, values written once
  uint32_t pending = n >= U ? ((1u << U) - 1u) : ((1u << (n > 0 ? n : 0)) - 1u);
#pragma unroll
  for (int u = 0; u < U; ++u) val[u] = 0u;
  uint32_t tries = 0;
  while (pending != 0u) {
    u64 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (pending & (1u << u)) v[u] = acquire ? ld_tag_acquire(addr(u)) : ld_tag(addr(u));
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if ((pending & (1u << u)) && (uint32_t)(v[u] >> 32) == tag) {
        val[u] = (uint32_t)v[u];
        pending &= ~(1u << u);
      }
    }
    if (pending != 0u && ((++tries) & 255u) == 0u) {
      const bool expired = tries >= c.poll_limit;
      if (expired) atomicCAS(reinterpret_cast<unsigned*>(c.status), 0u, 0x100u | (tag & 0xFFu));
      if (expired || ld_relaxed_u32(c.status) != 0u) {
        bad = true;
        return;
      }
    }
  }
}

// ---- one unit = (column, group): 128 weights ------------------------------------------------
__device__ __forceinline__ uint32_t h2_as_u32(half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

struct UnitF16 {
  half2 w[kWordsPerGroup][4];  // dequantised (q - zp) * s, pairs (i, i + 4) of every word
};
// Unit u of a region of U units -> 64 registers of fp16 weights.
__device__ __forceinline__ void load_unit(UnitF16& f, const unsigned char* region, int U, int u) {
  uint4 p[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) p[j] = *reinterpret_cast<const uint4*>(region + ((size_t)j * U + u) * 16);
  const uint32_t sz = *reinterpret_cast<const uint32_t*>(region + (size_t)64 * U + 4 * u);
  const half2 s2 = __half2half2(__ushort_as_half((unsigned short)(sz & 0xFFFFu)));
  const half2 zp = zp_to_half2((int)(sz >> 16));
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t ww[4] = {p[j].x, p[j].y, p[j].z, p[j].w};
#pragma unroll
    for (int t = 0; t < 4; ++t) dequant8(ww[t], zp, s2, f.w[4 * j + t]);
  }
}
// acc[m] = sum over the unit's group of w * x_m; xs points at the group's first k of row 0
// (perm8 order inside each slab of 8), rows `stride` halves apart.
template <int M>
__device__ __forceinline__ void unit_dot(const UnitF16& f, const half* xs, int stride, float (&acc)[M]) {
  float a4[M][4];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int q = 0; q < 4; ++q) a4[m][q] = 0.f;
#pragma unroll
  for (int j = 0; j < kWordsPerGroup; ++j) {
    // activation loads are not moved further ahead than four slabs: the weights already
    // occupy half of the register file
    if ((j & 3) == 0) asm volatile("" ::: "memory");
#pragma unroll
    for (int m = 0; m < M; ++m) dot8_h(f.w[j], xs + m * stride + 8 * j, a4[m]);
  }
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = (a4[m][0] + a4[m][1]) + (a4[m][2] + a4[m][3]);
}

// ---- residual stream -> RMSNorm ------------------------------------------------------------
// Thread t owns words t and t + 256 (elements 2w, 2w+1) of every row; xw[m][i] = the two halves
// of word t + 256 i (zero beyond word 447).  Writes the raw row to xraw (natural order) and the
// fp16-rounded normalised row to xn (perm8 order, or natural when `natural`).  Ends with a CTA
// barrier.  Returns true (for every thread) when any thread of the CTA came in with `bad` set;
// nothing useful has been written then.
template <int M>
__device__ __forceinline__ bool norm_rows(const uint32_t (&xw)[M][2], const uint32_t (&lnw)[2], float eps, bool natural,
                                          bool bad) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float ss[M];
#pragma unroll
  for (int m = 0; m < M; ++m) {
    ss[m] = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int w = tid + i * kPThreads;
      if (w < kXWords) {
        const float2 f = __half22float2(u32_as_half2(xw[m][i]));
        ss[m] += f.x * f.x + f.y * f.y;
        reinterpret_cast<uint32_t*>(XRAW)[m * kXWords + w] = xw[m][i];
      }
    }
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const float s = warp_sum(ss[m]);
    if (lane == 0) SSQ[m * 16 + warp] = s;
  }
  if (__syncthreads_or(bad ? 1 : 0)) return true;
#pragma unroll
  for (int m = 0; m < M; ++m) {
    float s = lane < kPWarps ? SSQ[m * 16 + lane] : 0.f;
    s = warp_sum(s);
    const float r = rsqrtf(s * (1.0f / kHidden) + eps);
    half* dst = XN + m * kHidden;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int w = tid + i * kPThreads;
      if (w < kXWords) {
        const float2 f = __half22float2(u32_as_half2(xw[m][i]));
        const float2 lw = __half22float2(u32_as_half2(lnw[i]));
        const half h0 = __float2half_rn(f.x * r * lw.x), h1 = __float2half_rn(f.y * r * lw.y);
        const int k = 2 * w;
        if (natural) {
          dst[k] = h0;
          dst[k + 1] = h1;
        } else {
          dst[perm_k(k)] = h0;
          dst[perm_k(k + 1)] = h1;
        }
      }
    }
  }
  __syncthreads();
  return false;
}

// ---- attention on 32 cached tokens per warp (fragment mappings as attn_warp.cuh) -----------
struct Tile32 {
  uint4 kr[4][2];  // K rows t0 + 8nb + g, bytes [32c, 32c + 32)
  uint4 vr[2][4];  // V rows t0 + 16j + 2c + {0,1,8,9}, dims 8g .. 8g+7
};
__device__ __forceinline__ void tile32_request(Tile32& t, const half* kbase, const half* vbase, int t0, int last,
                                               int g, int c) {
#pragma unroll
  for (int nb = 0; nb < 4; ++nb) {
    const half* kp = kbase + (size_t)min(t0 + 8 * nb + g, last) * kHeadDim + 16 * c;
    t.kr[nb][0] = ld_cg_u128(kp);
    t.kr[nb][1] = ld_cg_u128(kp + 8);
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int row = t0 + 16 * j + 2 * c + (r & 1) + 8 * (r >> 1);
      t.vr[j][r] = ld_cg_u128(vbase + (size_t)min(row, last) * kHeadDim + 8 * g);
    }
  }
}
// The row of the token being decoded comes from shared memory (knew, vnew: 64 halves each).
__device__ __forceinline__ void tile32_patch(Tile32& t, const half* knew, const half* vnew, int t0, int fresh,
                                             int g, int c) {
#pragma unroll
  for (int nb = 0; nb < 4; ++nb) {
    if (t0 + 8 * nb + g == fresh) {
      t.kr[nb][0] = *reinterpret_cast<const uint4*>(knew + 16 * c);
      t.kr[nb][1] = *reinterpret_cast<const uint4*>(knew + 16 * c + 8);
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int row = t0 + 16 * j + 2 * c + (r & 1) + 8 * (r >> 1);
      if (row == fresh) t.vr[j][r] = *reinterpret_cast<const uint4*>(vnew + 8 * g);
    }
  }
}
// m = row maximum of the scaled scores of tokens < len, l = sum of the fp16-rounded
// probabilities, o = sum of p * V (un-normalised); o[j][0], o[j][1] are dims 16c + j,
// 16c + 8 + j of head g.
__device__ __forceinline__ void tile32_attend(const Tile32& t, const uint32_t (&qa0)[4], const uint32_t (&qa2)[4],
                                              int t0, int len, float scale, int c, float& m_out, float& l_out,
                                              float (&o)[8][4]) {
  float sc[4][2];
  float m = -INFINITY;
  {
    float d[4][4];
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) d[nb][0] = d[nb][1] = d[nb][2] = d[nb][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
      for (int nb = 0; nb < 4; ++nb) {
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&t.kr[nb][0]);
        mma16816(d[nb], qa0[ks], 0u, qa2[ks], 0u, u[2 * ks], u[2 * ks + 1]);
      }
    }
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int tok = t0 + 8 * nb + 2 * c + e;
        const float v = tok < len ? d[nb][e] * scale : -INFINITY;
        sc[nb][e] = v;
        m = fmaxf(m, v);
      }
    }
  }
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
  uint32_t pa[2][2];
  float l = 0.f;
#pragma unroll
  for (int nb = 0; nb < 4; ++nb) {
    const float p0 = (sc[nb][0] == -INFINITY) ? 0.f : __expf(sc[nb][0] - m);
    const float p1 = (sc[nb][1] == -INFINITY) ? 0.f : __expf(sc[nb][1] - m);
    const half2 ph = __floats2half2_rn(p0, p1);
    l += __low2float(ph) + __high2float(ph);
    pa[nb >> 1][nb & 1] = *reinterpret_cast<const uint32_t*>(&ph);
  }
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
#pragma unroll
  for (int jk = 0; jk < 2; ++jk) {
    const uint32_t* r0 = reinterpret_cast<const uint32_t*>(&t.vr[jk][0]);
    const uint32_t* r1 = reinterpret_cast<const uint32_t*>(&t.vr[jk][1]);
    const uint32_t* r2 = reinterpret_cast<const uint32_t*>(&t.vr[jk][2]);
    const uint32_t* r3 = reinterpret_cast<const uint32_t*>(&t.vr[jk][3]);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint32_t b0_lo = __byte_perm(r0[w], r1[w], 0x5410), b0_hi = __byte_perm(r0[w], r1[w], 0x7632);
      const uint32_t b1_lo = __byte_perm(r2[w], r3[w], 0x5410), b1_hi = __byte_perm(r2[w], r3[w], 0x7632);
      mma16816(o[2 * w], pa[jk][0], 0u, pa[jk][1], 0u, b0_lo, b1_lo);
      mma16816(o[2 * w + 1], pa[jk][0], 0u, pa[jk][1], 0u, b0_hi, b1_hi);
    }
  }
  m_out = m;
  l_out = l;
}

// ---- weight ring ---------------------------------------------------------------------------
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// Bounded wait for a ring slot (about a second at most); false on timeout.
__device__ __forceinline__ bool ring_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 18); ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
// Requests the blob of global layer index q (= step * n_layers + layer) into ring slot q & 1.
__device__ __forceinline__ void ring_issue(const PersistArgs& a, int q, int cta, uint32_t ring_s, uint32_t bar_s) {
  const int layer = q % a.n_layers;
  const unsigned char* src = a.blobs + ((size_t)layer * kPCtas + cta) * kBlobStride;
  const uint32_t dst = ring_s + (uint32_t)(q & 1) * kBlobStride;
  const uint32_t bar = bar_s + 8u * (uint32_t)(q & 1);
  const uint32_t front = cta < kOCtas ? (uint32_t)kOffGu : (cta < kQkvCtas ? (uint32_t)kOffO : 0u);
  const uint32_t gu = (uint32_t)(gu_pairs_of(cta) * 4 * kGroupsH * kUnitBytes);
  mbar_expect_tx(bar, front + gu);
  if (front) bulk_g2s(dst, src, front, bar);
  bulk_g2s(dst + kOffGu, src + kOffGu, gu, bar);
}

struct Best {
  float v;
  int i;
};
__device__ __forceinline__ Best better(Best a, Best b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }
__device__ __forceinline__ Best warp_best(Best x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  return x;
}

template <int M>
__device__ __noinline__ bool phase_attn(uint32_t epoch, int layer, int q) {
  const SmArgs& sa = *reinterpret_cast<const SmArgs*>(smem_base + SL<M>::args);
  const PersistArgs& a = sa.a;
  Ctx c;
  c.status = reinterpret_cast<uint32_t*>(a.sync) + 1;
  c.poll_limit = sa.poll_limit;
  // Thread and CTA index pass through an opaque move: everything a phase derives from them is
  // then computed inside the phase instead of being hoisted out of the layer loop and kept in
  // registers for the whole kernel (which made the phases, inlined together, spill heavily).
  int tid_ = threadIdx.x, cta_ = blockIdx.x;
  asm volatile("" : "+r"(tid_), "+r"(cta_));
  const int tid = tid_, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
  const int cta = cta_;
  const int nb = a.batch < M ? a.batch : M;
  int* const s_pos = ST;
  int* const s_slot = ST + M;
  int* const s_tok = ST + 2 * M;
  const SyncLayout sl = sync_layout();
  bool bad = false;  // this thread gave up on a wait; folded into the next CTA barrier
  (void)warp; (void)lane; (void)gid; (void)tig; (void)s_pos; (void)s_slot; (void)s_tok; (void)sl; (void)nb;
  // The ring is only ever written by bulk copies, which the compiler does not see; without the
  // opaque offset below it moves the next phase's weight loads up into the previous phase and
  // then has to spill the 64 registers a unit occupies.
  uint32_t blob_off = (uint32_t)(q & 1) * kBlobStride;
  asm volatile("" : "+r"(blob_off) : : "memory");
  const unsigned char* blob = smem_base + SL<M>::ring + blob_off;
  const half* ln1 = a.lnw + (size_t)layer * 2 * kHidden;
  const half* ln2 = ln1 + kHidden;
  const size_t kv_plane = (size_t)a.n_slots * kKvHeads * a.s_max * kHeadDim;
  const size_t slot_stride = (size_t)kKvHeads * a.s_max * kHeadDim;
  half* kc = a.kv + (size_t)(2 * layer) * kv_plane;
  half* vc = kc + kv_plane;
  const int S = a.splits;
  (void)blob; (void)ln1; (void)ln2; (void)slot_stride; (void)kc; (void)vc; (void)S;
  // =========================== phase 2: attention splits =====================================
  {
    float* part = reinterpret_cast<float*>(SCR);                          // [15][7][66]
    half* qkvs = reinterpret_cast<half*>(SCR + kAttnPartBytes);  // [9][64], read with 16-byte loads
    const int n_tasks = nb * kKvHeads * S;
    for (int task = cta; task < n_tasks; task += kPCtas) {
      const int m = task / (kKvHeads * S), rem = task % (kKvHeads * S);
      const int kvh = rem / S, sp = rem % S;
      const int pos = s_pos[m], len = pos + 1;
      const int t_begin = sp * a.chunk;
      const int t0 = t_begin + 32 * warp;
      const bool active = 32 * warp < a.chunk && t0 < len;
      const half* kbase = kc + (size_t)s_slot[m] * slot_stride + (size_t)kvh * a.s_max * kHeadDim;
      const half* vbase = vc + (size_t)s_slot[m] * slot_stride + (size_t)kvh * a.s_max * kHeadDim;
      Tile32 tile;
      if (active) tile32_request(tile, kbase, vbase, t0, pos > 0 ? pos - 1 : 0, gid, tig);
      {
        // the 7 query heads of the group, then the key and the value of the token: 288 words
        uint32_t w[2];
        auto head_of = [&](int t) {
          const int hh = t >> 5;
          return hh < 7 ? kvh * 7 + hh : (hh == 7 ? kHeads + kvh : kHeads + kKvHeads + kvh);
        };
        poll_words<2>(c, [&](int u) {
          const int t = tid + u * kPThreads;
          return QKVX + (size_t)m * kQkvWords + head_of(t) * 32 + (t & 31);
        }, tid + kPThreads < 288 ? 2 : 1, make_tag(epoch, layer, kTagQkv), w, bad);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int t = tid + u * kPThreads;
          if (t < 288) {
            const half2 h = u32_as_half2(w[u]);
            qkvs[(t >> 5) * kHeadDim + (t & 31)] = __low2half(h);
            qkvs[(t >> 5) * kHeadDim + (t & 31) + 32] = __high2half(h);
          }
        }
      }
      if (__syncthreads_or(bad ? 1 : 0)) return false;
      if (active) {
        uint32_t qa0[4], qa2[4];
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          qa0[ks] = qa2[ks] = 0u;
          if (gid < 7) {
            const uint2 u = *reinterpret_cast<const uint2*>(qkvs + gid * kHeadDim + 16 * tig + 4 * ks);
            qa0[ks] = u.x;
            qa2[ks] = u.y;
          }
        }
        tile32_patch(tile, qkvs + 7 * kHeadDim, qkvs + 8 * kHeadDim, t0, pos, gid, tig);
        float mw, lw, o[8][4];
        tile32_attend(tile, qa0, qa2, t0, len, 0.125f, tig, mw, lw, o);
        if (gid < 7) {
          float* dst = part + (warp * 7 + gid) * 66;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            dst[16 * tig + j] = o[j][0];
            dst[16 * tig + 8 + j] = o[j][1];
          }
          if (tig == 0) {
            dst[64] = mw;
            dst[65] = lw;
          }
        }
      }
      __syncthreads();
      {
        // merge this CTA's warps, publish one partial per (row, kv head, split)
        int nw = len - t_begin;
        nw = nw > a.chunk ? a.chunk : nw;
        nw = nw > 0 ? (nw + 31) >> 5 : 0;
#pragma unroll 1
        for (int t = tid; t < 7 * kHeadDim; t += kPThreads) {
        const int h = t >> 6, d = t & 63;
        float mx = -INFINITY;
        for (int w = 0; w < nw; ++w) mx = fmaxf(mx, part[(w * 7 + h) * 66 + 64]);
        float den = 0.f, num = 0.f;
        if (mx != -INFINITY) {
          for (int w = 0; w < nw; ++w) {
            const float mwv = part[(w * 7 + h) * 66 + 64];
            const float e = mwv == -INFINITY ? 0.f : __expf(mwv - mx);
            den += e * part[(w * 7 + h) * 66 + 65];
            num += e * part[(w * 7 + h) * 66 + d];
          }
        }
        u64* dst = ATTX + ((size_t)(m * kKvHeads + kvh) * kPMaxSplits + sp) * kAttWords + h * 66;
        const uint32_t tag = make_tag(epoch, layer, kTagAtt);
        st_tag(dst + d, __float_as_uint(num), tag);
        if (d == 0) st_tag(dst + 64, __float_as_uint(mx), tag);
        if (d == 1) st_tag(dst + 65, __float_as_uint(den), tag);
        }
      }
      __syncthreads();
    }
  }
  return true;
}

// The four linears of a layer as ONE loop body (kind 0 qkv, 1 o_proj, 2 gate|up, 3 down), so
// the register-heavy code exists once.  A thread owns up to two units (units tid and tid + 256):
// 128 registers of dequantised weights held across the poll of the phase's input.  The kernel
// runs 8 warps per SM so that every thread has 255 registers: nothing may spill, a spill costs a
// round trip to L2 here because almost all of the SM's L1 is carved out as shared memory.
// The attention phase runs between kind 0 and kind 1 on the CTAs that own an attention task.
template <int M>
__device__ __forceinline__ bool layer_phases(uint32_t epoch, int layer, int q) {
  const SmArgs& sa = *reinterpret_cast<const SmArgs*>(smem_base + SL<M>::args);
  const PersistArgs& a = sa.a;
  Ctx c;
  c.status = reinterpret_cast<uint32_t*>(a.sync) + 1;
  c.poll_limit = sa.poll_limit;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, cta = blockIdx.x;
  const int nb = a.batch < M ? a.batch : M;
  int* const s_pos = ST;
  int* const s_slot = ST + M;
  int* const s_tok = ST + 2 * M;
  const SyncLayout sl = sync_layout();
  bool bad = false;  // this thread gave up on a wait; folded into the next CTA barrier
  const unsigned char* blob = smem_base + SL<M>::ring + (size_t)(q & 1) * kBlobStride;
  const int gu_pairs = gu_pairs_of(cta), gu_pair0 = gu_pair0_of(cta);
  const int gu_cols = 2 * gu_pairs, gu_units = gu_cols * 2 * kGroupsH;

#pragma unroll 1
  for (int kind = 0; kind < 4; ++kind) {
    if (kind == 1 && cta < nb * kKvHeads * a.splits) {
      if (!phase_attn<M>(epoch, layer, q)) return false;
    }
    // ---- this CTA's units of the linear: (column, group), units tid and tid + 256
    const bool cta_on = kind == 0 ? cta < kQkvCtas : (kind == 2 ? true : cta < kOCtas);
    const int U = !cta_on ? 0 : (kind == 2 ? gu_units : (kind == 3 ? kUnitsD : kUnitsH));
    const int off = kind == 0 ? kOffQkv : (kind == 1 ? kOffO : (kind == 2 ? kOffGu : kOffDown));
    UnitF16 wf[kUnitsPerThread];
#pragma unroll
    for (int i = 0; i < kUnitsPerThread; ++i)
      if (tid + i * kPThreads < U) load_unit(wf[i], blob + off, U, tid + i * kPThreads);
    if (kind == 3) {
      // every warp has taken what it needs from this layer's blob: refill the slot
      __syncthreads();
      if (tid == 0 && q + 2 < a.steps * a.n_layers) {
        fence_proxy_async();
        ring_issue(a, q + 2, cta, smem_u32(smem_base + SL<M>::ring), smem_u32(smem_base + SL<M>::bars));
        ST[3 * M] = q + 3;  // blobs requested so far (thread 0's book-keeping)
      }
    }
    if (!cta_on) continue;

    // ---- qkv epilogue inputs: requested now, converted only in the epilogue
    const int em = tid >> 2, ei = tid & 3;  // (row, column pair) of an 8-column CTA's epilogue
    const int n0 = 8 * cta + 2 * ei, head = n0 >> 6, pj = (n0 & 63) >> 1;
    half2 bias_h = __floats2half2_rn(0.f, 0.f);
    half cs_h = __float2half(1.f), sn_h = __float2half(0.f);
    int epos = 0;
    if (kind == 0 && tid < 4 * nb) {
      bias_h = *reinterpret_cast<const half2*>(blob + kOffBias + 4 * ei);
      epos = s_pos[em];
      if (head < kHeads + kKvHeads) {
        const int p = epos < a.max_pos ? epos : a.max_pos - 1;
        cs_h = a.cos_t[(size_t)p * 32 + pj];
        sn_h = a.sin_t[(size_t)p * 32 + pj];
      }
    }

    // ---- input of the linear -> shared memory (perm8 order)
    const half* xs = XN;
    int stride = kHidden;
    if (kind == 0 || kind == 2) {
      // residual stream -> RMSNorm: thread owns words tid and tid + 256 of every row
      const half* ln = a.lnw + ((size_t)layer * 2 + (kind == 2 ? 1 : 0)) * kHidden;
      const int nwords = tid + kPThreads < kXWords ? 2 : 1;
      uint32_t lnw[2];
      lnw[0] = ldg_nc_u32(ln + 2 * tid);
      lnw[1] = nwords > 1 ? ldg_nc_u32(ln + 2 * (tid + kPThreads)) : 0u;
      uint32_t xw[M][2];
#pragma unroll
      for (int m = 0; m < M; ++m) {
        xw[m][0] = xw[m][1] = 0u;
        if (m < nb) {
          if (kind == 0 && layer == 0) {
            int tk = s_tok[m];
            tk = tk < 0 ? 0 : (tk >= a.vocab ? a.vocab - 1 : tk);
            xw[m][0] = ldg_nc_u32(a.embed + (size_t)tk * kHidden + 2 * tid);
            if (nwords > 1) xw[m][1] = ldg_nc_u32(a.embed + (size_t)tk * kHidden + 2 * (tid + kPThreads));
          } else {
            const u64* src = (kind == 0 ? XA : XB) + (size_t)m * kXWords;
            poll_words<2>(c, [&](int u) { return src + tid + u * kPThreads; }, nwords,
                          make_tag(epoch, layer, kind == 0 ? kTagX : kTagXb), xw[m], bad);
          }
        }
      }
      if (norm_rows<M>(xw, lnw, a.eps, false, bad)) return false;
    } else if (kind == 1) {
      // merge the attention splits: item = (head qh, dims 2j, 2j+1), items tid and tid + 256
      const uint32_t tag = make_tag(epoch, layer, kTagAtt);
      const int S = a.splits;
#pragma unroll 1
      for (int it = tid; it < kXWords; it += kPThreads) {
        const int qh = it >> 5, j = it & 31;
        const int kvh = qh / 7, h = qh % 7;
#pragma unroll 1
        for (int m = 0; m < nb; ++m) {
          float v0 = 0.f, v1 = 0.f;
          float mx = -INFINITY, den = 0.f, n0s = 0.f, n1s = 0.f;
          const u64* base = ATTX + ((size_t)(m * kKvHeads + kvh) * kPMaxSplits) * kAttWords + h * 66;
          for (int s0 = 0; s0 < S; s0 += 4) {
            uint32_t w[16];
            const int n = S - s0 >= 4 ? 16 : 4 * (S - s0);
            poll_words<16>(c, [&](int u) {
              const int which = u & 3;
              const int o = which == 0 ? 2 * j : (which == 1 ? 2 * j + 1 : (which == 2 ? 64 : 65));
              return base + (size_t)(s0 + (u >> 2)) * kAttWords + o;
            }, n, tag, w, bad);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (s0 + e < S) {
                const float ms = __uint_as_float(w[4 * e + 2]), ls = __uint_as_float(w[4 * e + 3]);
                if (ms != -INFINITY) {
                  const float mn = fmaxf(mx, ms);
                  const float keep = mx == -INFINITY ? 0.f : __expf(mx - mn);
                  const float ex = __expf(ms - mn);
                  den = den * keep + ex * ls;
                  n0s = n0s * keep + ex * __uint_as_float(w[4 * e]);
                  n1s = n1s * keep + ex * __uint_as_float(w[4 * e + 1]);
                  mx = mn;
                }
              }
            }
          }
          if (mx != -INFINITY && den > 0.f) {
            v0 = n0s / den;
            v1 = n1s / den;
          }
          // the attention output is an fp16 tensor in the reference
          half* dst = XN + m * kHidden;
          dst[perm_k(qh * 64 + 2 * j)] = __float2half_rn(v0);
          dst[perm_k(qh * 64 + 2 * j + 1)] = __float2half_rn(v1);
        }
      }
      if (__syncthreads_or(bad ? 1 : 0)) return false;
    } else {
      // SwiGLU output of all CTAs -> shared memory: thread owns words tid + 256 u
      half* acts = reinterpret_cast<half*>(SCR);
      const uint32_t tag = make_tag(epoch, layer, kTagAct);
#pragma unroll 1
      for (int m = 0; m < nb; ++m) {
        uint32_t w[10];
        const int n = (kActWords - tid + kPThreads - 1) / kPThreads;  // 10 or 9
        poll_words<10>(c, [&](int u) { return ACTX + (size_t)m * kActWords + tid + u * kPThreads; }, n, tag, w, bad);
#pragma unroll
        for (int u = 0; u < 10; ++u) {
          if (u < n) {
            const int k = 2 * (tid + u * kPThreads);
            const half2 h = u32_as_half2(w[u]);
            acts[m * kInter + perm_k(k)] = __low2half(h);
            acts[m * kInter + perm_k(k + 1)] = __high2half(h);
          }
        }
      }
      if (__syncthreads_or(bad ? 1 : 0)) return false;
      xs = acts;
      stride = kInter;
    }

    // ---- 128 weights x M rows per unit, partial sums to shared memory
#pragma unroll
    for (int i = 0; i < kUnitsPerThread; ++i) {
      const int u = tid + i * kPThreads;
      if (u < U) {
        const int group = kind == 2 ? (u / gu_cols) >> 1 : u >> 3;
        float acc[M];
        unit_dot<M>(wf[i], xs + group * kGroup, stride, acc);
#pragma unroll
        for (int m = 0; m < M; ++m) RED[m * kRedStride + u] = acc[m];
      }
    }
    __syncthreads();

    // ---- epilogue: sum over the groups, round as the reference does, publish
    if (kind == 2) {
      if (tid < gu_pairs * nb) {
        const int gm = tid / gu_pairs, gi = tid - gm * gu_pairs;  // row, column pair of this CTA
        float g0 = 0.f, g1 = 0.f, u0 = 0.f, u1 = 0.f;
#pragma unroll
        for (int g = 0; g < kGroupsH; ++g) {
          const float* pg = RED + gm * kRedStride + (2 * g) * gu_cols + 2 * gi;
          const float* pu = pg + gu_cols;
          g0 += pg[0];
          g1 += pg[1];
          u0 += pu[0];
          u1 += pu[1];
        }
        // gate and up are fp16 linear outputs in the reference; SwiGLU output is fp16 too
        const float a0 = silu_mul(__half2float(__float2half_rn(g0)), __half2float(__float2half_rn(u0)));
        const float a1 = silu_mul(__half2float(__float2half_rn(g1)), __half2float(__float2half_rn(u1)));
        st_tag(ACTX + (size_t)gm * kActWords + gu_pair0 + gi, h2_as_u32(__floats2half2_rn(a0, a1)),
               make_tag(epoch, layer, kTagAct));
      }
    } else if (tid < 4 * nb) {
      const int ng = kind == 3 ? kGroupsI : kGroupsH;
      float v0 = 0.f, v1 = 0.f;
#pragma unroll 2
      for (int g = 0; g < ng; ++g) {
        v0 += RED[em * kRedStride + g * 8 + 2 * ei];
        v1 += RED[em * kRedStride + g * 8 + 2 * ei + 1];
      }
      if (kind == 0) {
        // fp16 linear output with bias, as the reference's GEMM writes it
        const float2 bias2 = __half22float2(bias_h);
        const float cs = __half2float(cs_h), sn = __half2float(sn_h);
        v0 = __half2float(__float2half_rn(v0 + bias2.x));
        v1 = __half2float(__float2half_rn(v1 + bias2.y));
        float lo = v0, hi = v1;  // dims pj and pj + 32 of the head
        if (head < kHeads + kKvHeads) {
          lo = v0 * cs - v1 * sn;
          hi = v0 * sn + v1 * cs;
        }
        const half lo16 = __float2half_rn(lo), hi16 = __float2half_rn(hi);
        st_tag(QKVX + (size_t)em * kQkvWords + head * 32 + pj, h2_as_u32(__halves2half2(lo16, hi16)),
               make_tag(epoch, layer, kTagQkv));
        if (head >= kHeads && epos < a.s_max) {
          const size_t kv_plane = (size_t)a.n_slots * kKvHeads * a.s_max * kHeadDim;
          const int kvh = (head - kHeads) & 1;
          half* base = a.kv + (size_t)(2 * layer + (head < kHeads + kKvHeads ? 0 : 1)) * kv_plane;
          half* row = base + ((size_t)s_slot[em] * kKvHeads + kvh) * a.s_max * kHeadDim + (size_t)epos * kHeadDim;
          row[pj] = lo16;
          row[pj + 32] = hi16;
        }
      } else {
        // residual add: the row this CTA's columns came in with is still in shared memory
        const float2 r = __half22float2(*reinterpret_cast<const half2*>(XRAW + em * kHidden + 8 * cta + 2 * ei));
        const half x0 = __float2half_rn(r.x + __half2float(__float2half_rn(v0)));
        const half x1 = __float2half_rn(r.y + __half2float(__float2half_rn(v1)));
        if (kind == 1) {
          if (!(cta == 0 && layer == sa.withhold_layer))
            st_tag(XB + (size_t)em * kXWords + 4 * cta + ei, h2_as_u32(__halves2half2(x0, x1)),
                   make_tag(epoch, layer, kTagXb));
        } else {
          st_tag(XA + (size_t)em * kXWords + 4 * cta + ei, h2_as_u32(__halves2half2(x0, x1)),
                 make_tag(epoch, layer + 1, kTagX));
        }
      }
    }
  }
  (void)lane; (void)warp;
  return true;
}

template <int M>
__device__ __noinline__ bool phase_lm_head(uint32_t epoch, int step) {
  const SmArgs& sa = *reinterpret_cast<const SmArgs*>(smem_base + SL<M>::args);
  const PersistArgs& a = sa.a;
  Ctx c;
  c.status = reinterpret_cast<uint32_t*>(a.sync) + 1;
  c.poll_limit = sa.poll_limit;
  // Thread and CTA index pass through an opaque move: everything a phase derives from them is
  // then computed inside the phase instead of being hoisted out of the layer loop and kept in
  // registers for the whole kernel (which made the phases, inlined together, spill heavily).
  int tid_ = threadIdx.x, cta_ = blockIdx.x;
  asm volatile("" : "+r"(tid_), "+r"(cta_));
  const int tid = tid_, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
  const int cta = cta_;
  const int nb = a.batch < M ? a.batch : M;
  int* const s_pos = ST;
  int* const s_slot = ST + M;
  int* const s_tok = ST + 2 * M;
  const SyncLayout sl = sync_layout();
  bool bad = false;  // this thread gave up on a wait; folded into the next CTA barrier
  (void)warp; (void)lane; (void)gid; (void)tig; (void)s_pos; (void)s_slot; (void)s_tok; (void)sl; (void)nb;
  const int step0 = sa.step0;
  // =========================== final norm -> tied lm_head -> argmax ===========================
  {
    const int npairs = a.vocab >> 1;
    const int p_begin = (int)((int64_t)npairs * cta / kPCtas);
    const int p_end = (int)((int64_t)npairs * (cta + 1) / kPCtas);
    constexpr int kVec = 7;  // 16-byte pieces of a row pair per lane
    int dim[kVec];
#pragma unroll
    for (int j = 0; j < kVec; ++j) dim[j] = ((lane + 32 * j) % (kHidden / 8)) * 8;
    uint4 wa[kVec], wb[kVec];
    int p = p_begin + 2 * warp;
    auto request = [&](int pp) {
      const uint4* s0 = reinterpret_cast<const uint4*>(a.embed + (size_t)(pp < p_end ? pp : p_begin) * 2 * kHidden);
      const uint4* s1 = reinterpret_cast<const uint4*>(a.embed + (size_t)(pp + 1 < p_end ? pp + 1 : p_begin) * 2 * kHidden);
#pragma unroll
      for (int j = 0; j < kVec; ++j) wa[j] = ldg_nc_u128(s0 + lane + 32 * j);
#pragma unroll
      for (int j = 0; j < kVec; ++j) wb[j] = ldg_nc_u128(s1 + lane + 32 * j);
    };
    request(p);  // first rows of the table before the hidden state is there
    const int nwords = tid + kPThreads < kXWords ? 2 : 1;
    uint32_t lnw[2];
    lnw[0] = ldg_nc_u32(a.final_norm + 2 * tid);
    lnw[1] = nwords > 1 ? ldg_nc_u32(a.final_norm + 2 * (tid + kPThreads)) : 0u;
    uint32_t xw[M][2];
#pragma unroll
    for (int m = 0; m < M; ++m) {
      xw[m][0] = xw[m][1] = 0u;
      if (m < nb)
        poll_words<2>(c, [&](int u) { return XA + (size_t)m * kXWords + tid + u * kPThreads; }, nwords,
                      make_tag(epoch, a.n_layers, kTagX), xw[m], bad);
    }
    if (norm_rows<M>(xw, lnw, a.eps, true, bad)) return false;
    const half* xh = XN;
    uint4 xr[M == 1 ? kVec : 1];
    if (M == 1) {
#pragma unroll
      for (int j = 0; j < kVec; ++j) xr[M == 1 ? j : 0] = *reinterpret_cast<const uint4*>(xh + dim[j]);
    }
    Best best[M];
#pragma unroll
    for (int m = 0; m < M; ++m) {
      best[m].v = -INFINITY;
      best[m].i = 0x7fffffff;
    }
    auto consume = [&](int pp, const uint4 (&wv)[kVec]) {
      float acc0[M], acc1[M];
#pragma unroll
      for (int m = 0; m < M; ++m) acc0[m] = acc1[m] = 0.f;
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        const half2* w2 = reinterpret_cast<const half2*>(&wv[j]);
        const bool first = (j < 3) || (j == 3 && lane < 16);  // pieces 0..111 are the pair's first row
#pragma unroll
        for (int m = 0; m < M; ++m) {
          uint4 xv;
          if (M == 1) xv = xr[M == 1 ? j : 0];
          else xv = *reinterpret_cast<const uint4*>(xh + m * kHidden + dim[j]);
          const half2* x2 = reinterpret_cast<const half2*>(&xv);
          float s0 = 0.f, s1 = 0.f;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s0 = fma_h(s0, __low2half(w2[e]), __low2half(x2[e]));
            s1 = fma_h(s1, __high2half(w2[e]), __high2half(x2[e]));
          }
          if (first) acc0[m] += s0 + s1; else acc1[m] += s0 + s1;
        }
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float l0 = __half2float(__float2half_rn(warp_sum(acc0[m])));
        const float l1 = __half2float(__float2half_rn(warp_sum(acc1[m])));
        if (a.logits != nullptr && lane == 0 && m < nb)
          *reinterpret_cast<half2*>(a.logits + (size_t)m * a.vocab + 2 * pp) = __floats2half2_rn(l0, l1);
        Best cnd;
        cnd.v = l0;
        cnd.i = 2 * pp;
        best[m] = better(best[m], cnd);
        cnd.v = l1;
        cnd.i = 2 * pp + 1;
        best[m] = better(best[m], cnd);
      }
    };
    while (p < p_end) {
      consume(p, wa);
      if (p + 1 < p_end) consume(p + 1, wb);
      p += 2 * kPWarps;
      if (p < p_end) request(p);
    }
    // CTA best per row -> candidates of all CTAs -> the same argmax in every CTA
    float* bv_s = RED;                                     // [M][16]
    int* bi_s = reinterpret_cast<int*>(RED + M * 16);      // [M][16]
#pragma unroll
    for (int m = 0; m < M; ++m) {
      if (lane == 0) {
        bv_s[m * 16 + warp] = best[m].v;
        bi_s[m * 16 + warp] = best[m].i;
      }
    }
    __syncthreads();
    const uint32_t ctag = make_tag(epoch, a.n_layers, kTagCand);
    if (warp < nb) {
      Best cb;
      cb.v = lane < kPWarps ? bv_s[warp * 16 + lane] : -INFINITY;
      cb.i = lane < kPWarps ? bi_s[warp * 16 + lane] : 0x7fffffff;
      cb = warp_best(cb);
      if (lane == 0) {
        // release: the K/V rows this CTA appended during the token become visible to every
        // CTA that reads this candidate (they attend to those rows from the next token on)
        st_tag_release(CANDX + ((size_t)cta * kPMaxRows + warp) * 2, __float_as_uint(cb.v), ctag);
        st_tag_release(CANDX + ((size_t)cta * kPMaxRows + warp) * 2 + 1, (uint32_t)cb.i, ctag);
      }
    }
    float* cv_s = reinterpret_cast<float*>(SCR);                   // [M][148]
    int* ci_s = reinterpret_cast<int*>(SCR + M * kPCtas * 4);      // [M][148]
#pragma unroll 1
    for (int item = tid; item < 2 * kPCtas; item += kPThreads) {
      uint32_t w[M];
      const int src = item >> 1, which = item & 1;
      poll_words<M>(c, [&](int u) { return CANDX + ((size_t)src * kPMaxRows + u) * 2 + which; }, nb, ctag, w, bad,
                    true);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        if (which == 0) cv_s[m * kPCtas + src] = __uint_as_float(w[m]);
        else ci_s[m * kPCtas + src] = (int)w[m];
      }
    }
    if (__syncthreads_or(bad ? 1 : 0)) return false;
    if (warp < nb) {
      Best cb;
      cb.v = -INFINITY;
      cb.i = 0x7fffffff;
      for (int i = lane; i < kPCtas; i += 32) {
        Best d;
        d.v = cv_s[warp * kPCtas + i];
        d.i = ci_s[warp * kPCtas + i];
        cb = better(cb, d);
      }
      cb = warp_best(cb);
      if (lane == 0) {
        const int token = cb.i == 0x7fffffff ? 0 : cb.i;
        s_tok[warp] = token;
        const int newpos = s_pos[warp] + 1;
        s_pos[warp] = newpos;
        if (cta == 0) {
          const int slot = s_slot[warp];
          a.tok[slot] = token;
          a.pos[slot] = newpos;
          if (a.out_tokens != nullptr)
            a.out_tokens[(size_t)((step0 + step) % a.ring) * a.n_slots + slot] = token;
        }
      }
    }
    __syncthreads();
    if (cta == 0 && tid == 0 && a.step_counter != nullptr) {
      __threadfence();  // tokens and positions are visible before the step counter moves
      *a.step_counter = step0 + step + 1;
    }
  }
  return true;
}

template <int M>
__global__ void __launch_bounds__(kPThreads, 1) token_kernel(const PersistArgs a) {
  const int tid = threadIdx.x, cta = blockIdx.x;
  const int nb = a.batch < M ? a.batch : M;
  const uint32_t ring_s = smem_u32(smem_base + SL<M>::ring), bar_s = smem_u32(smem_base + SL<M>::bars);
  int* const s_pos = ST;
  int* const s_slot = ST + M;
  int* const s_tok = ST + 2 * M;
  SmArgs& sa = *reinterpret_cast<SmArgs*>(smem_base + SL<M>::args);
  uint32_t* const status = reinterpret_cast<uint32_t*>(a.sync) + 1;

  // header of the exchange area: [0] epoch, [1] status, [2] probes per poll before it gives
  // up (0 = default), [3] test hook: CTA 0 withholds its o_proj result of layer [3] - 1
  const uint32_t* hdr = reinterpret_cast<const uint32_t*>(a.sync);
  const uint32_t epoch0 = ld_relaxed_u32(hdr);
  const int total_q = a.steps * a.n_layers;
  if (tid == 0) {
    mbar_init(bar_s, 1);
    mbar_init(bar_s + 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // the phases read the launch arguments from shared memory
    sa.a = a;
    sa.poll_limit = ld_relaxed_u32(hdr + 2) != 0u ? ld_relaxed_u32(hdr + 2) : kPollLimit;
    sa.withhold_layer = (int)ld_relaxed_u32(hdr + 3) - 1;
    sa.step0 = a.step_counter != nullptr ? *a.step_counter : 0;
    ring_issue(a, 0, cta, ring_s, bar_s);
    if (total_q > 1) ring_issue(a, 1, cta, ring_s, bar_s);
    ST[3 * M] = total_q > 1 ? 2 : 1;
    ST[3 * M + 1] = 0;  // no wait has given up yet
  }
  if (tid < M) {
    int slot = 0, p = 0, t = 0;
    if (tid < nb) {
      slot = a.rows[tid];
      slot = slot < 0 ? 0 : (slot >= a.n_slots ? a.n_slots - 1 : slot);
      p = a.pos[slot];
      t = a.tok[slot];
    }
    s_slot[tid] = slot;
    s_pos[tid] = p;
    s_tok[tid] = t;
  }
  __syncthreads();

  uint32_t epoch = epoch0;
  bool alive = true;
  int q = 0;
  int n_waited = 0;  // blobs whose arrival every thread of the CTA has waited for
  for (int step = 0; step < a.steps && alive; ++step) {
    epoch = next_epoch(epoch);
    for (int layer = 0; layer < a.n_layers && alive; ++layer, ++q) {
      bool late = false;
      if (!ring_wait(bar_s + 8u * (uint32_t)(q & 1), (uint32_t)((q >> 1) & 1))) {
        atomicCAS(reinterpret_cast<unsigned*>(status), 0u, 0x200u);
        late = true;
      }
      n_waited = q + 1;
      if (__syncthreads_or(late ? 1 : 0)) {
        alive = false;
        break;
      }
      alive = layer_phases<M>(epoch, layer, q);
    }
    if (!alive) break;
    alive = phase_lm_head<M>(epoch, step);
  }

  // ---- orderly exit: nothing of this CTA's copies may still be in flight -----------------------
  __syncthreads();
  if (tid == 0) {
    for (int w = n_waited; w < ST[3 * M]; ++w) ring_wait(bar_s + 8u * (uint32_t)(w & 1), (uint32_t)((w >> 1) & 1));
    // The epochs an abandoned burst may have touched are spent: some CTAs can be one token
    // ahead of this one when a wait gives up, and their tags must never be valid again.
    if (cta == 0) *reinterpret_cast<uint32_t*>(a.sync) = alive ? epoch : next_epoch(next_epoch(epoch));
  }
}

// ---- W4T -> W4S stream -------------------------------------------------------------------------
struct PackArgs {
  quic_w4_t qkv, o, gu, down;
  const half* ln1;
  const half* ln2;
  unsigned char* blobs;  // this layer: [148][kBlobStride]
  half* lnw;             // this layer: [2][896]
};
// One thread per (unit, piece): piece 0..3 = four packed words, piece 4 = {scale, zero point}.
__device__ __forceinline__ void pack_unit(unsigned char* region, int U, int u, const quic_w4_t& w, int n, int g,
                                          int piece) {
  if (piece < 4) {
    const int32_t* p = w.qw + ((size_t)g * kWordsPerGroup + 4 * piece) * w.n + n;
    uint4 v;
    v.x = (uint32_t)p[0];
    v.y = (uint32_t)p[(size_t)w.n];
    v.z = (uint32_t)p[(size_t)2 * w.n];
    v.w = (uint32_t)p[(size_t)3 * w.n];
    *reinterpret_cast<uint4*>(region + ((size_t)piece * U + u) * 16) = v;
  } else {
    const unsigned short sc = __half_as_ushort(reinterpret_cast<const half*>(w.sc)[(size_t)g * w.n + n]);
    const uint32_t zb = w.zp[(size_t)g * (w.n >> 1) + (n >> 1)];
    const uint32_t zp = (zb >> (4 * (n & 1))) & 15u;
    *reinterpret_cast<uint32_t*>(region + (size_t)64 * U + 4 * u) = (uint32_t)sc | (zp << 16);
  }
}

// grid (148, 4 linears), block 512: thread = unit, loops over the five pieces.
__global__ void __launch_bounds__(512) persist_pack_kernel(const PackArgs a) {
  const int cta = blockIdx.x, which = blockIdx.y, t = threadIdx.x;
  unsigned char* blob = a.blobs + (size_t)cta * kBlobStride;
  for (int piece = 0; piece < 5; ++piece) {
    if (which == 0 && cta < kQkvCtas && t < kUnitsH)
      pack_unit(blob + kOffQkv, kUnitsH, t, a.qkv, 8 * cta + (t & 7), t >> 3, piece);
    if (which == 1 && cta < kOCtas && t < kUnitsH)
      pack_unit(blob + kOffO, kUnitsH, t, a.o, 8 * cta + (t & 7), t >> 3, piece);
    if (which == 2 && cta < kOCtas && t < kUnitsD)
      pack_unit(blob + kOffDown, kUnitsD, t, a.down, 8 * cta + (t & 7), t >> 3, piece);
    if (which == 3) {
      const int cols = 2 * gu_pairs_of(cta), units = cols * 2 * kGroupsH;
      if (t < units) {
        const int blk = t / cols, col = t - blk * cols;
        const int n = ((blk & 1) ? kInter : 0) + 2 * gu_pair0_of(cta) + col;
        pack_unit(blob + kOffGu, units, t, a.gu, n, blk >> 1, piece);
      }
    }
  }
  if (which == 0 && cta < kQkvCtas && t < 8)
    reinterpret_cast<half*>(blob + kOffBias)[t] =
        a.qkv.bias ? reinterpret_cast<const half*>(a.qkv.bias)[8 * cta + t] : __float2half(0.f);
  if (cta == 0 && which == 0) {
    for (int i = t; i < kHidden; i += 512) {
      a.lnw[i] = a.ln1[i];
      a.lnw[kHidden + i] = a.ln2[i];
    }
  }
}

inline int64_t stream_header_bytes(int n_layers) { return ((int64_t)n_layers * 2 * kHidden * 2 + 255) / 256 * 256; }

template <int M>
int launch_token_kernel(const PersistArgs& pa, cudaStream_t st) {
  static bool configured[64] = {};
  int dev = 0;
  QUIC_CUDA(cudaGetDevice(&dev));
  constexpr int smem = SL<M>::total;
  if (dev < 64 && !configured[dev]) {
    int sms = 0, coop = 0;
    QUIC_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    QUIC_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    QUIC_REQUIRE(sms >= kPCtas && coop != 0, QUIC_E_SHAPE,
                 "decode_persist: needs 148 SMs and cooperative launch (every CTA must be resident)");
    QUIC_CUDA(cudaFuncSetAttribute(token_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    int per_sm = 0;
    QUIC_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, token_kernel<M>, kPThreads, smem));
    QUIC_REQUIRE(per_sm >= 1, QUIC_E_SHAPE, "decode_persist: the kernel does not fit an SM");
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kPCtas);
  cfg.blockDim = dim3(kPThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  QUIC_CUDA(cudaLaunchKernelEx(&cfg, token_kernel<M>, pa));
  return QUIC_OK;
}

}  // namespace
}  // namespace quic

using namespace quic;

extern "C" int32_t quic_persist_max_rows(void) { return kPMaxRows; }

extern "C" int64_t quic_persist_stream_bytes(int32_t n_layers) {
  if (n_layers < 1 || n_layers > kPMaxLayers) return 0;
  return stream_header_bytes(n_layers) + (int64_t)n_layers * kPCtas * kBlobStride;
}

extern "C" int64_t quic_persist_sync_bytes(void) { return sync_layout().total; }

extern "C" int32_t quic_persist_pick_splits(int32_t batch, int32_t ctx) {
  if (ctx < 1) ctx = 1;
  if (batch < 1) batch = 1;
  // A split is at most 256 tokens (one 32-token tile per warp).  Short contexts are still cut
  // in up to four so that no SM has to pull more than ~50 KB of cache per layer; the o_proj
  // CTAs merge the splits themselves, which costs them 4 polled words per split.
  int s = (ctx + 32 * kPWarps - 1) / (32 * kPWarps);
  int want = (ctx + 191) / 192;
  if (want > 4) want = 4;
  if (s < want) s = want;
  return s;  // > kPMaxSplits: the context is too long for this kernel
}

extern "C" int quic_persist_pack(const quic_model_t* m, void* stream_out, void* stream) {
  QUIC_REQUIRE(m && stream_out, QUIC_E_ARG, "persist_pack: null argument");
  QUIC_REQUIRE(m->n_layers >= 1 && m->n_layers <= kPMaxLayers && m->layers, QUIC_E_SHAPE,
               "persist_pack: 1..30 layers");
  QUIC_REQUIRE((uintptr_t)stream_out % 256 == 0, QUIC_E_ARG, "persist_pack: output must be 256-byte aligned");
  unsigned char* base = static_cast<unsigned char*>(stream_out);
  const int64_t hdr = stream_header_bytes(m->n_layers);
  QUIC_CUDA(cudaMemsetAsync(base, 0, (size_t)quic_persist_stream_bytes(m->n_layers), (cudaStream_t)stream));
  for (int l = 0; l < m->n_layers; ++l) {
    const quic_layer_t& L = m->layers[l];
    QUIC_REQUIRE(L.qkv.n == kQkvN && L.qkv.k == kHidden && L.o.n == kHidden && L.o.k == kHidden &&
                     L.gate_up.n == 2 * kInter && L.gate_up.k == kHidden && L.down.n == kHidden &&
                     L.down.k == kInter,
                 QUIC_E_SHAPE, "persist_pack: layer shapes are not Qwen2.5-0.5B's");
    QUIC_REQUIRE(L.qkv.qw && L.o.qw && L.gate_up.qw && L.down.qw && L.ln1 && L.ln2, QUIC_E_ARG,
                 "persist_pack: missing layer tensor");
    PackArgs pa;
    pa.qkv = L.qkv;
    pa.o = L.o;
    pa.gu = L.gate_up;
    pa.down = L.down;
    pa.ln1 = (const half*)L.ln1;
    pa.ln2 = (const half*)L.ln2;
    pa.blobs = base + hdr + (size_t)l * kPCtas * kBlobStride;
    pa.lnw = reinterpret_cast<half*>(base) + (size_t)l * 2 * kHidden;
    persist_pack_kernel<<<dim3(kPCtas, 4), 512, 0, (cudaStream_t)stream>>>(pa);
    QUIC_CUDA(cudaGetLastError());
  }
  return QUIC_OK;
}

extern "C" int quic_decode_persist(const quic_model_t* m, const quic_decode_t* d, const void* wstream, void* sync,
                                   int32_t steps, void* stream) {
  QUIC_REQUIRE(m && d && wstream && sync, QUIC_E_ARG, "decode_persist: null argument");
  QUIC_REQUIRE(m->n_layers >= 1 && m->n_layers <= kPMaxLayers, QUIC_E_SHAPE, "decode_persist: 1..30 layers");
  QUIC_REQUIRE(m->vocab >= 2 * kPCtas && m->vocab % 2 == 0, QUIC_E_SHAPE,
               "decode_persist: even vocabulary of at least 296 rows");
  QUIC_REQUIRE(m->embed && m->final_norm && m->rope_cos && m->rope_sin && m->max_pos >= 1, QUIC_E_ARG,
               "decode_persist: missing model tensor");
  QUIC_REQUIRE(d->kv && d->tok && d->pos && d->rows, QUIC_E_ARG, "decode_persist: missing state tensor");
  QUIC_REQUIRE(d->batch >= 1 && d->batch <= kPMaxRows, QUIC_E_LIMIT, "decode_persist: 1..4 batch rows");
  QUIC_REQUIRE(d->n_slots >= 1 && d->s_max >= 1, QUIC_E_SHAPE, "decode_persist: bad cache geometry");
  QUIC_REQUIRE(steps >= 1 && steps <= 4096, QUIC_E_ARG, "decode_persist: 1..4096 steps");
  QUIC_REQUIRE(d->out_tokens == nullptr || (d->ring >= 1 && d->step_counter != nullptr), QUIC_E_ARG,
               "decode_persist: out_tokens needs ring >= 1 and a step counter");
  QUIC_REQUIRE(d->logits == nullptr || steps == 1, QUIC_E_ARG, "decode_persist: logits are kept for one step only");
  QUIC_REQUIRE((uintptr_t)wstream % 256 == 0 && (uintptr_t)sync % 256 == 0, QUIC_E_ARG,
               "decode_persist: stream and sync area must be 256-byte aligned");
  int ctx = d->ctx_hint > 0 ? d->ctx_hint : d->s_max;
  if (ctx > d->s_max) ctx = d->s_max;
  const int splits = d->attn_splits > 0 ? d->attn_splits : quic_persist_pick_splits(d->batch, ctx);
  QUIC_REQUIRE(splits <= kPMaxSplits, QUIC_E_LIMIT, "decode_persist: context too long (more than 16 splits)");
  int chunk = ((ctx + splits - 1) / splits + 31) / 32 * 32;
  QUIC_REQUIRE(chunk <= 32 * kPWarps, QUIC_E_LIMIT, "decode_persist: a split would exceed 256 tokens");
  PersistArgs pa = {};
  const unsigned char* base = static_cast<const unsigned char*>(wstream);
  pa.blobs = base + stream_header_bytes(m->n_layers);
  pa.lnw = reinterpret_cast<const half*>(base);
  pa.embed = (const half*)m->embed;
  pa.final_norm = (const half*)m->final_norm;
  pa.cos_t = (const half*)m->rope_cos;
  pa.sin_t = (const half*)m->rope_sin;
  pa.n_layers = m->n_layers;
  pa.vocab = m->vocab;
  pa.max_pos = m->max_pos;
  pa.eps = m->eps;
  pa.kv = (half*)d->kv;
  pa.n_slots = d->n_slots;
  pa.s_max = d->s_max;
  pa.tok = d->tok;
  pa.pos = d->pos;
  pa.rows = d->rows;
  pa.batch = d->batch;
  pa.out_tokens = d->out_tokens;
  pa.ring = d->ring > 0 ? d->ring : 1;
  pa.step_counter = d->step_counter;
  pa.logits = (half*)d->logits;
  pa.sync = static_cast<unsigned char*>(sync);
  pa.steps = steps;
  pa.splits = splits;
  pa.chunk = chunk;
  cudaStream_t st = (cudaStream_t)stream;
  if (d->batch <= 1) return launch_token_kernel<1>(pa, st);
  if (d->batch <= 2) return launch_token_kernel<2>(pa, st);
  return launch_token_kernel<4>(pa, st);
}

extern "C" int quic_decode_persist_status(void* sync, void* stream, int32_t* status_out) {
  QUIC_REQUIRE(sync && status_out, QUIC_E_ARG, "decode_persist_status: null argument");
  cudaStream_t st = (cudaStream_t)stream;
  uint32_t v = 0;
  unsigned char* word = static_cast<unsigned char*>(sync) + 4;
  QUIC_CUDA(cudaMemcpyAsync(&v, word, 4, cudaMemcpyDeviceToHost, st));
  QUIC_CUDA(cudaStreamSynchronize(st));
  if (v != 0) QUIC_CUDA(cudaMemsetAsync(word, 0, 4, st));  // nothing else runs on the area meanwhile
  *status_out = (int32_t)v;
  return QUIC_OK;
}

extern "C" int quic_decode_persist_run_host(const quic_model_t* m, const quic_decode_t* d, const void* wstream,
                                            void* sync, int32_t steps, void* stream, const int32_t* host_in,
                                            int32_t* dev_in, int32_t n_in, const int32_t* dev_out,
                                            int32_t* host_out, int32_t n_out, int32_t* host_status) {
  QUIC_REQUIRE(n_in >= 0 && n_out >= 0, QUIC_E_ARG, "decode_persist_run_host: negative count");
  QUIC_REQUIRE(n_in == 0 || (host_in != nullptr && dev_in != nullptr), QUIC_E_ARG,
               "decode_persist_run_host: null input buffer");
  QUIC_REQUIRE(n_out == 0 || (host_out != nullptr && dev_out != nullptr), QUIC_E_ARG,
               "decode_persist_run_host: null output buffer");
  QUIC_REQUIRE(host_status != nullptr && sync != nullptr, QUIC_E_ARG, "decode_persist_run_host: null status buffer");
  cudaStream_t st = (cudaStream_t)stream;
  if (n_in > 0) QUIC_CUDA(cudaMemcpyAsync(dev_in, host_in, sizeof(int32_t) * n_in, cudaMemcpyHostToDevice, st));
  const int rc = quic_decode_persist(m, d, wstream, sync, steps, stream);
  if (rc != QUIC_OK) return rc;
  if (n_out > 0)
    QUIC_CUDA(cudaMemcpyAsync(host_out, dev_out, sizeof(int32_t) * n_out, cudaMemcpyDeviceToHost, st));
  QUIC_CUDA(cudaMemcpyAsync(host_status, static_cast<const unsigned char*>(sync) + 4, 4, cudaMemcpyDeviceToHost, st));
  QUIC_CUDA(cudaStreamSynchronize(st));
  if (*host_status != 0) {
    QUIC_CUDA(cudaMemsetAsync(static_cast<unsigned char*>(sync) + 4, 0, 4, st));
    return fail(QUIC_E_TIMEOUT, "decode_persist: a bounded wait inside the kernel gave up; the tokens of this call are invalid");
  }
  return QUIC_OK;
}
