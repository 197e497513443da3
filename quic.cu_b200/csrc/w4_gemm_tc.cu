// W4A16 GEMM (two rows and more) on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   y[m, n] = sum_k x[m, k] * dequant(W)[n, k] (+ bias[n])      fp16 in/out, fp32 accumulate
//
// Replaces the reference's Marlin kernel (kernels/cuda/marlin.cu:1527, reached through
// src/quant/marlin.py:190) at the batch sizes where it tiles mma.sync; nothing of its
// structure is kept.  Mapping ("swap AB"): the 128 weight rows of a CTA tile sit on the
// M side of the UMMA (TMEM lanes), the batch rows on its N side (TMEM columns), so the
// accumulator of a 128 x MT tile is MT fp32 columns of tensor memory and a thread of the
// epilogue owns one output column n.
//
// Per pipeline stage (128 of K = one quantisation group = two 128-byte swizzle atoms)
//   1. the TMA warp brings the packed tile (16 int32 words per weight row) and the x tiles
//      (MT rows x 128 bytes per atom, swizzled by TMA) into shared memory;
//   2. 16 warps dequantise the packed words exactly like the GEMV path ((q - zp) * s rounded
//      once to fp16) and write each row's bytes into the A tiles in the K-major 128-byte
//      swizzled layout the UMMA shared-memory descriptor expects, make the writes visible
//      to the async proxy and arrive on the stage's barrier;
//   3. one thread issues the stage's tcgen05.mma (K = 16 each) that accumulate into TMEM and,
//      where the stage will be refilled, commits them to the stage's "empty" mbarrier.
// Split-K CTAs write fp32 partials that the consumer kernel (or a small finish kernel) sums;
// the gate|up form applies SwiGLU in its epilogue.  Every mbarrier wait is bounded: on a
// timeout the kernel records an error code, still frees its tensor memory and returns.
#include "tc_common.cuh"

namespace quic {
namespace {

constexpr int kCounterInts = 4096;  // arrival counters at the head of the split-K workspace

// Error words of the tensor path: [0] the GEMM, [1] the tensor lm_head.  0 = ok; otherwise
// (code << 16) | block of the first bounded wait that gave up.
__device__ int g_tc_status[2];

// What a test may change for the launches that follow (quic_w4a16_tensor_test_hook): the probe
// limit of the bounded waits and one k block whose packed weight tile the producer never requests.
uint32_t g_spin_limit = kSpinLimit;
int g_skip_kblock = -1;

struct GemmArgs {
  quic_w4_t w;
  half* y;         // [m_total, N]    (splits == 1)
  float* part;     // [splits, m_total, N] fp32 (splits > 1)
  int* counters;   // one per (n tile, m tile), zero on entry, left zero
  int m_total;
  int kblocks_per_split;
  int mtl;     // batch-row tiles per CTA (2 from 129 rows up)
  uint32_t spin_limit;  // probes of a bounded wait
  int skip_kblock;      // test hook: the weight tile of this k block is never requested (-1: none)
  // SwiGLU fused into the epilogue of the gate|up linear: the CTA's 128 weight rows are 64
  // gate rows and the 64 up rows of the same columns (two 64-row TMA boxes per stage), and y
  // is the activation [m_total, N / 2] = silu(gate) * up.
  int fuse_swiglu;
};

constexpr int kConsumers = 512;                 // 16 warps dequantise (4 per scheduler) and run the epilogue
constexpr int kGemmThreads = kConsumers + 64;   // + TMA warp + MMA warp (one lane each)
// A pipeline stage covers kSub swizzle atoms of K (2 x 64 = 128 = one quantisation group): the
// fixed per-stage costs of every role (a barrier round trip, a fence, a commit) are paid
// half as often as with one atom per stage.
// Many rows over a short K (prefill: K = 896 is seven groups) turn this around: a CTA's prologue
// and epilogue weigh as much as its main loop and a two-stage ring leaves the loads' latency
// exposed, so there a stage is ONE atom (KS = 1), a CTA holds two of them, and two CTAs share
// an SM -- one CTA's epilogue runs under the other's main loop.
constexpr int kSub = 2;
constexpr int kStageK = kBlockK * kSub;
// Scales (fp16) and zero points (a nibble) of a stage's 128 weight rows travel with the stage.
constexpr uint32_t kScBytes = kTileN * 2, kZpBytes = kTileN / 2, kScArea = 1024;

// MTL = batch-row tiles per CTA: one dequantised weight tile feeds MTL MMAs groups, so the
// dequantisation work per flop drops MTL-fold (large M: prefill).
template <int MT, int MTL = 1, int KS = kSub>
struct Smem {
  static constexpr uint32_t kRaw = 8 * KS * kTileN * 4;                   // packed tile: 8 KS k-words x 128 rows
  static constexpr uint32_t kBTile = ((uint32_t)MT * 128u + 1023u) & ~1023u;  // one x tile (MT rows x 64 k), swizzled by TMA
  static constexpr uint32_t kB = kBTile * MTL * KS;
  static constexpr uint32_t kASub = kTileN * 128;                        // dequantised 128 rows x 64 k
  static constexpr uint32_t kA = kASub * KS;
  static constexpr uint32_t kStage = kRaw + kB + kA + kScArea;        // [packed | x tiles | A | scales, zero points]
  // as many stages as fit
  static constexpr int kStages = (int)((210u * 1024u) / kStage) > 4 ? 4 : (int)((210u * 1024u) / kStage);
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Roles.  Warp 16, lane 0: streams (packed weight tile, x tile) pairs through a TMA ring.
// Warps 0-15: turn each packed tile into the swizzled fp16 A operand of its stage and tell
// the MMA warp (one mbarrier arrival per warp).  Warp 17, lane 0: issues the MMAs of a stage
// once its A tile is complete and commits them to the stage's "empty" barrier, which lets
// the TMA warp refill it.  No role ever waits for another role's instruction issue, only
// for data.  Warps 0-15 read the accumulator back at the end.
template <int MT, int kStages, int MTL, int KS>
__global__ void __launch_bounds__(kGemmThreads) w4a16_gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w,
                                                                     const __grid_constant__ CUtensorMap tm_x,
                                                                     const GemmArgs a) {
  using L = Smem<MT, MTL, KS>;
  constexpr int kMaxStages = kStages;
  constexpr int kSub = KS;                   // (shadows the default: atoms per stage of THIS kernel)
  constexpr int kStageK = kBlockK * KS;
  constexpr uint32_t kRawBytes = L::kRaw;
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kMaxStages];    // packed weight tile landed (TMA bytes)
  __shared__ __align__(8) uint64_t bar_aready[kMaxStages];  // 16 consumer warps finished the A tile AND the x tile landed
  __shared__ __align__(8) uint64_t bar_empty[kMaxStages];   // MMAs that read the stage completed
  __shared__ __align__(8) uint64_t bar_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int fail_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * kTileN;
  const int split = blockIdx.y;
  const int m0 = blockIdx.z * MT * MTL;
  const int N = a.w.n;
  const int kb_total = a.w.k / kStageK;
  const int kb0 = split * a.kblocks_per_split;
  const int kb1 = min(kb_total, kb0 + a.kblocks_per_split);
  const int nkb = kb1 - kb0;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));

  constexpr uint32_t kCols = MT * MTL < 32 ? 32 : MT * MTL;  // power of two >= 32
  if (tid == 0) {
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_aready[s]), kConsumers / 32 + 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_done), 1);
    fail_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_base_s)),
                 "r"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  const int half_n = N >> 1;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = tmem_base_s;
  const uint32_t idesc = umma_idesc_f16(MT);
  // Everything above touched weights and on-chip state only.  The activations (and the
  // buffers the epilogue writes) belong to the previous kernels of the stream: the producer
  // requests the packed weight tiles of the first ring pass, THEN waits for the predecessor
  // and requests the x tiles; the other roles wait before they touch global memory.
  pdl_launch_dependents();

  if (warp == kConsumers / 32) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      const int first = nkb < kStages ? nkb : kStages;
      // weight side of k block `kb` into the stage at raw_s: packed tile, scales, zero points
      const half* scp = reinterpret_cast<const half*>(a.w.sc);
      auto load_weights = [&](uint32_t raw_s, int kb, uint32_t full) {
        const uint32_t sc_s = raw_s + L::kStage - kScArea, zp_s = sc_s + kScBytes;
        const size_t g = (size_t)((kb * kStageK) / kGroup);
        mbar_expect_tx(full, kRawBytes + kScBytes + kZpBytes);
        if (a.fuse_swiglu) {  // two boxes of 64 rows: gate rows, then the up rows of the same columns
          const int ng = (int)blockIdx.x * 64, nu = half_n + ng;
          tma_load_2d(raw_s, &tm_w, ng, kb * 8 * kSub, full);
          tma_load_2d(raw_s + kRawBytes / 2, &tm_w, nu, kb * 8 * kSub, full);
          bulk_load(sc_s, scp + g * N + ng, kScBytes / 2, full);
          bulk_load(sc_s + kScBytes / 2, scp + g * N + nu, kScBytes / 2, full);
          bulk_load(zp_s, a.w.zp + g * half_n + (ng >> 1), kZpBytes / 2, full);
          bulk_load(zp_s + kZpBytes / 2, a.w.zp + g * half_n + (nu >> 1), kZpBytes / 2, full);
        } else {
          tma_load_2d(raw_s, &tm_w, n0, kb * 8 * kSub, full);
          bulk_load(sc_s, scp + g * N + n0, kScBytes, full);
          bulk_load(zp_s, a.w.zp + g * half_n + (n0 >> 1), kZpBytes, full);
        }
      };
      for (int it = 0; it < first; ++it) {
        if (kb0 + it == a.skip_kblock) continue;  // test hook: the consumers' wait for this tile runs out
        load_weights(base + it * L::kStage, kb0 + it, smem_u32(&bar_full[it]));
      }
      pdl_wait();
      for (int it = 0; it < first; ++it) {
        const uint32_t xfull = smem_u32(&bar_aready[it]);
        mbar_expect_tx(xfull, (uint32_t)MT * 128u * MTL * kSub);
#pragma unroll
        for (int i = 0; i < MTL * kSub; ++i)  // tile i: rows of row tile i / kSub, k atom i % kSub; rows past the end read as zero
          tma_load_2d(base + it * L::kStage + kRawBytes + i * L::kBTile, &tm_x,
                      ((kb0 + it) * kSub + i % kSub) * kBlockK, m0 + (i / kSub) * MT, xfull);
      }
      // (ring position and phase are carried along: the depth is a run-time value)
      for (int it = first, stage = 0, pass = 1; it < nkb; ++it) {
        if (!mbar_wait(smem_u32(&bar_empty[stage]), (pass - 1) & 1, a.spin_limit)) {
          fail_s = 2;
          break;
        }
        const uint32_t raw_s = base + stage * L::kStage, b_s = raw_s + kRawBytes;
        const uint32_t full = smem_u32(&bar_full[stage]), xfull = smem_u32(&bar_aready[stage]);
        if (kb0 + it != a.skip_kblock) load_weights(raw_s, kb0 + it, full);  // (test hook: see the first pass)
        mbar_expect_tx(xfull, (uint32_t)MT * 128u * MTL * kSub);
#pragma unroll
        for (int i = 0; i < MTL * kSub; ++i)
          tma_load_2d(b_s + i * L::kBTile, &tm_x, ((kb0 + it) * kSub + i % kSub) * kBlockK, m0 + (i / kSub) * MT, xfull);
        if (++stage == kStages) {
          stage = 0;
          ++pass;
        }
      }
    }
  } else if (warp == kConsumers / 32 + 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // One wait per k block (operand A written by the consumer warps and operand B landed by
      // TMA arrive on the same barrier) and a commit only where somebody waits for it: each
      // of these costs the issuing thread a round trip, and at these sizes the loop is bound
      // by that, not by the tensor pipe.
      for (int it = 0, stage = 0, pass = 0; it < nkb; ++it) {
        if (!mbar_wait(smem_u32(&bar_aready[stage]), pass & 1, a.spin_limit)) {
          fail_s = 3;
          break;
        }
        if (it == 0) tc_fence_after();
        const uint32_t b_s = base + stage * L::kStage + kRawBytes, a_s = b_s + L::kB;
#pragma unroll
        for (int i = 0; i < MTL; ++i) {
          if (i > 0 && m0 + i * MT >= a.m_total) break;  // tile of rows beyond the end
#pragma unroll
          for (int sub = 0; sub < kSub; ++sub)
#pragma unroll
            for (int k = 0; k < kBlockK / 16; ++k)
              umma_f16(tmem_d + (uint32_t)(i * MT), umma_desc_sw128(a_s + sub * L::kASub + k * 32),
                       umma_desc_sw128(b_s + (i * kSub + sub) * L::kBTile + k * 32), idesc,
                       (it > 0 || sub > 0 || k > 0) ? 1u : 0u);
        }
        if (it + kStages < nkb) umma_commit(smem_u32(&bar_empty[stage]));
        if (it == nkb - 1) umma_commit(smem_u32(&bar_done));
        if (++stage == kStages) {
          stage = 0;
          ++pass;
        }
      }
    }
  } else {
    // ---------------- consumers: dequantise ----------------
    const int row = tid & (kTileN - 1), part = tid >> 7;  // thread -> (row, four of its sixteen k-words)
    for (int it = 0, stage = 0, pass = 0; it < nkb; ++it) {
      // "full" of this phase also means the MMAs of the stage's previous use are complete
      // (the TMA warp refilled it only after "empty"), so the A tile may be overwritten.
      if (!mbar_wait(smem_u32(&bar_full[stage]), pass & 1, a.spin_limit)) {
        fail_s = 1;
        break;
      }
      unsigned char* stage_g = gen_base + stage * L::kStage;
      const uint32_t* raw_g = reinterpret_cast<const uint32_t*>(stage_g);
      unsigned char* a_g = stage_g + kRawBytes + L::kB;
      const half* sc_s = reinterpret_cast<const half*>(stage_g + L::kStage - kScArea);
      const uint8_t* zp_s = reinterpret_cast<const uint8_t*>(sc_s) + kScBytes;  // byte r / 2: rows r (low nibble), r + 1
      const half2 s2 = __half2half2(sc_s[row]);
      const half2 zp = zp_to_half2((zp_s[row >> 1] >> (4 * (row & 1))) & 15);
#pragma unroll
      for (int jj = 0; jj < 2 * kSub; ++jj) {
        const int j = 2 * kSub * part + jj;  // k-word 0..15 of the stage: atom j / 8, 16-byte chunk j % 8
        half2 d[4];
        // packed word j of tile row `row`: one [16][128] box, or two [16][64] boxes
        const int raw_i = a.fuse_swiglu ? (row >> 6) * (8 * kSub * 64) + j * 64 + (row & 63) : j * kTileN + row;
        dequant8(raw_g[raw_i], zp, s2, d);  // d[p] = (k = p, k = p + 4)
        const uint32_t u0 = *reinterpret_cast<uint32_t*>(&d[0]), u1 = *reinterpret_cast<uint32_t*>(&d[1]);
        const uint32_t u2 = *reinterpret_cast<uint32_t*>(&d[2]), u3 = *reinterpret_cast<uint32_t*>(&d[3]);
        uint4 o;
        o.x = __byte_perm(u0, u1, 0x5410);  // (k0, k1)
        o.y = __byte_perm(u2, u3, 0x5410);  // (k2, k3)
        o.z = __byte_perm(u0, u1, 0x7632);  // (k4, k5)
        o.w = __byte_perm(u2, u3, 0x7632);  // (k6, k7)
        *reinterpret_cast<uint4*>(a_g + (j >> 3) * L::kASub + sw128_offset(row, j & 7)) = o;
      }
      fence_proxy_async();  // generic-proxy stores -> visible to the tensor core's async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_aready[stage]));
      if (++stage == kStages) {
        stage = 0;
        ++pass;
      }
    }
  }
  __syncwarp();

  // wait for the whole accumulation, then read the accumulator out of tensor memory
  if (warp < kConsumers / 32) {
    pdl_wait();  // the output / partial buffers may still be read by earlier kernels of the chain
    bool ok = !fail_s && nkb > 0;
    if (ok) ok = mbar_wait_relaxed(smem_u32(&bar_done), 0, 64, a.spin_limit);
    ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below is warp-collective
    tc_fence_after();
    if (!ok && tid == 0 && nkb > 0) atomicCAS(&g_tc_status[0], 0, ((fail_s ? fail_s : 3) << 16) | (int)blockIdx.x);
    constexpr int kOutCols = MT * MTL;       // accumulator columns = batch rows of the CTA
    constexpr int kWarpCols = kOutCols / 4;  // per warp of a lane quarter
    if (a.y != nullptr && gridDim.y == 1) {
      // A finished fp16 output (no K split): every warp reads its lane quarter kWarpCols / 2 columns at
      // a time, the CTA's output tile is put together in shared memory -- the operand ring is free
      // once the accumulation is complete -- and leaves in 16-byte pieces, whole 128- or 256-byte
      // rows at a time.  All 16 warps reach every barrier whether or not their waits succeeded.
      constexpr int kHalf = kWarpCols / 2;  // 2 (16 batch rows per CTA) .. 32 (256)
      const int quarter = warp & 3, cgroup = warp >> 2;  // cgroup: a quarter of the columns (= batch rows)
      const uint32_t lane_addr = tmem_d + ((uint32_t)(quarter * 32) << 16);
      float v[kHalf];
      if (a.fuse_swiglu) {
        // TMEM lanes 0-63 hold the gate rows, 64-127 the up rows of the same 64 activation columns.
        // Of a warp's batch rows the up warps hand the first half to the gate warps and the gate
        // warps the second half to the up warps (fp16-rounded, as the linear's output), so that
        // every warp finishes silu(gate) * up for half of them.
        float* ex = reinterpret_cast<float*>(gen_base);                            // [kOutCols][64] fp32
        half* out_s = reinterpret_cast<half*>(gen_base + kOutCols * 64 * sizeof(float));  // [kOutCols][64] fp16
        const bool up = quarter >= 2;
        const int row = (quarter & 1) * 32 + lane;  // 0..63 inside the gate (or up) half
        const int c_send = cgroup * kWarpCols + (up ? 0 : kHalf), c_fin = cgroup * kWarpCols + (up ? kHalf : 0);
        if (ok && m0 + c_send < a.m_total) {
          tmem_ld_cols<kHalf>(lane_addr + (uint32_t)c_send, v);
#pragma unroll
          for (int j = 0; j < kHalf; ++j) ex[(c_send + j) * 64 + row] = __half2float(__float2half_rn(v[j]));
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory");
        if (ok && m0 + c_fin < a.m_total) {
          tmem_ld_cols<kHalf>(lane_addr + (uint32_t)c_fin, v);
#pragma unroll
          for (int j = 0; j < kHalf; ++j) {
            const float mine = __half2float(__float2half_rn(v[j])), other = ex[(c_fin + j) * 64 + row];
            out_s[(c_fin + j) * 64 + row] = __float2half_rn(up ? silu_mul(other, mine) : silu_mul(mine, other));
          }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory");
        if (ok) {
#pragma unroll 1
          for (int id = tid; id < kOutCols * 8; id += kConsumers) {  // (batch row, 16-byte piece of its 128 bytes)
            const int t = id >> 3, piece = id & 7, m = m0 + t;
            if (m < a.m_total)
              *reinterpret_cast<uint4*>(a.y + (size_t)m * half_n + (size_t)blockIdx.x * 64 + piece * 8) =
                  *reinterpret_cast<const uint4*>(out_s + t * 64 + piece * 8);
          }
        }
      } else {
        half* out_s = reinterpret_cast<half*>(gen_base);  // [kOutCols][128] fp16
        const int col_l = quarter * 32 + lane;
        const bool has_bias = a.w.bias != nullptr;
        const float bias = has_bias ? __half2float(reinterpret_cast<const half*>(a.w.bias)[n0 + col_l]) : 0.f;
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {
          const int c0 = cgroup * kWarpCols + hh * kHalf;
          if (ok && m0 + c0 < a.m_total) {
            tmem_ld_cols<kHalf>(lane_addr + (uint32_t)c0, v);
#pragma unroll
            for (int j = 0; j < kHalf; ++j) {
              float o = __half2float(__float2half_rn(v[j]));
              if (has_bias) o += bias;
              out_s[(c0 + j) * kTileN + col_l] = __float2half_rn(o);
            }
          }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory");
        if (ok) {
#pragma unroll 1
          for (int id = tid; id < kOutCols * 16; id += kConsumers) {  // (batch row, 16-byte piece of its 256 bytes)
            const int t = id >> 4, piece = id & 15, m = m0 + t;
            if (m < a.m_total)
              *reinterpret_cast<uint4*>(a.y + (size_t)m * N + n0 + piece * 8) =
                  *reinterpret_cast<const uint4*>(out_s + t * kTileN + piece * 8);
          }
        }
      }
    } else if (ok) {
      // fp32 partial sums of this K split for a fused consumer.  TMEM lane = tile row; a warp may
      // read lanes 32*(warp % 4)..+31, so the four warps that share a lane quarter split the batch
      // columns between them and read theirs in one go.
      const int quarter = warp & 3, cgroup = warp >> 2;
      const int col = n0 + quarter * 32 + lane;
      constexpr int kPer = MT >= 32 ? MT / 4 : 8;
#pragma unroll 1
      for (int i = 0; i < MTL; ++i) {
        const int c0 = i * MT + cgroup * kPer;  // accumulator column = tile * MT + row inside the tile
        if (cgroup * kPer >= MT || m0 + c0 >= a.m_total) continue;
        float v[kPer];
        tmem_ld_cols<kPer>(tmem_d + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
          const int m = m0 + c0 + j;
          if (m < a.m_total) a.part[((size_t)split * a.m_total + m) * N + col] = v[j];
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(kCols) : "memory");
}

// Sums the split-K partials (one thread per four consecutive output elements, all loads in
// flight together), rounds to fp16 as the un-split epilogue does and adds the bias.
// N is a multiple of 128, so a group of four never straddles a row.
__global__ void tc_splitk_finish_kernel(const float* __restrict__ part, const half* __restrict__ bias,
                                        half* __restrict__ y, int m_total, int N, int splits) {
  const size_t idx = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const size_t total = (size_t)m_total * N;
  pdl_launch_dependents();
  pdl_wait();
  if (idx >= total) return;
  float4 p[16];
#pragma unroll
  for (int s = 0; s < 16; ++s)
    p[s] = s < splits ? __ldcg(reinterpret_cast<const float4*>(part + (size_t)s * total + idx))
                      : make_float4(0.f, 0.f, 0.f, 0.f);
  float4 v = p[0];
#pragma unroll
  for (int s = 1; s < 16; ++s) {
    v.x += p[s].x;
    v.y += p[s].y;
    v.z += p[s].z;
    v.w += p[s].w;
  }
  half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
  if (bias) {
    const half2* b2 = reinterpret_cast<const half2*>(bias + idx % N);
    const float2 l = __half22float2(lo), h = __half22float2(hi), bl = __half22float2(b2[0]), bh = __half22float2(b2[1]);
    lo = __floats2half2_rn(l.x + bl.x, l.y + bl.y);
    hi = __floats2half2_rn(h.x + bh.x, h.y + bh.y);
  }
  uint2 out;
  out.x = *reinterpret_cast<const uint32_t*>(&lo);
  out.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(y + idx) = out;
}

template <int MT, int kDeep, int MTL, int KS>
int run_variant(const half* x, GemmArgs a, int splits, cudaStream_t st) {
  using L = Smem<MT, MTL, KS>;
  CUtensorMap tm_w, tm_x;
  // packed weights int32 [K/8, N]: box = 8 KS k-words x 128 rows; x fp16 [m, K]: box = MT rows x 64 k,
  // written with the 128-byte swizzle the UMMA descriptor expects (rows past m read as zero)
  // (fused SwiGLU: two boxes of 64 rows per stage, gate rows and up rows)
  int rc = make_map(&tm_w, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, a.w.qw, (uint64_t)a.w.k / 8, (uint64_t)a.w.n, 8 * KS,
                    a.fuse_swiglu ? kTileN / 2 : kTileN, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != QUIC_OK) return rc;
  rc = make_map(&tm_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x, (uint64_t)a.m_total, (uint64_t)a.w.k, MT, kBlockK,
                CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != QUIC_OK) return rc;
  a.kblocks_per_split *= kSub / KS;  // planned in stages of kSub atoms
  const int mtiles = (a.m_total + MT - 1) / MT;
  const size_t smem = (size_t)kDeep * L::kStage + 1024;
  dim3 grid(a.w.n / kTileN, splits, (mtiles + MTL - 1) / MTL);
  QUIC_CUDA(cudaFuncSetAttribute(w4a16_gemm_tc_kernel<MT, kDeep, MTL, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem));
  QUIC_CUDA(launch(w4a16_gemm_tc_kernel<MT, kDeep, MTL, KS>, grid, dim3(kGemmThreads), smem, st, true, tm_w, tm_x, a));
  return QUIC_OK;
}

template <int MT>
int run(const half* x, const GemmArgs& args, int splits, cudaStream_t st) {
  GemmArgs a = args;
  a.spin_limit = g_spin_limit;
  a.skip_kblock = g_skip_kblock;
  if (a.mtl == 2) {
    if constexpr (MT == 128) {
      // Two CTAs per SM (2 x 53 KB, one-atom stages) when their waves take less time than the
      // waves of one CTA per SM: a CTA that shares its SM was measured at 1.86 x the time of one
      // that has it alone over a long K (4864) and about 1.5 x over a short one (896), where
      // prologue and epilogue weigh more -- e.g. 896 CTAs are 7 waves of 148 or 4 of 296.
      const int ctas = (a.w.n / kTileN) * (((a.m_total + MT - 1) / MT + 1) / 2);
      const int waves1 = (ctas + 147) / 148, waves2 = (ctas + 295) / 296;
      static_assert(2 * (2 * Smem<MT, 2, 1>::kStage + 2048) <= 227 * 1024 && Smem<MT, 2, 1>::kStages >= 2,
                    "two CTAs of two one-atom stages must fit one SM");
      if (splits == 1 && g_skip_kblock < 0 && waves2 * (a.w.k <= 1024 ? 150 : 186) <= waves1 * 100)
        return run_variant<MT, 2, 2, 1>(x, a, splits, st);
      return run_variant<MT, Smem<MT, 2>::kStages, 2, kSub>(x, a, splits, st);
    }
  }
  return run_variant<MT, Smem<MT>::kStages, 1, kSub>(x, a, splits, st);
}

}  // namespace

static void tc_plan(int m, int n, int k, int* mt_out, int* splits_out, int* per_out, int* mtl_out = nullptr) {
  const int kb_total = k / kStageK;
  const int tiles = n / kTileN;
  const int mt = m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128;
  const int mtiles = (m + mt - 1) / mt;
  // two row tiles share one dequantised weight tile once there is more than a wave of CTAs
  const int mtl = (mtiles >= 2 && tiles * mtiles > 148) ? 2 : 1;
  const int ctas = tiles * ((mtiles + mtl - 1) / mtl);
  // split K while it at most fills the SMs once, at most 16 ways, at least one stage per CTA
  int splits = 1;
  while (splits < 16 && ctas * splits * 2 <= 148 && kb_total / (splits * 2) >= 1) splits *= 2;
  int per = (kb_total + splits - 1) / splits;
  // a short K (seven stages) in single stages while that still fits one wave: the loop's length,
  // not the work, bounds a small GEMM
  // (64-row step 889 -> 881 us, 32 rows 781 -> 758)
  if (per == 2 && ctas * kb_total <= 148) per = 1;
  *mt_out = mt;
  *per_out = per;
  *splits_out = (kb_total + per - 1) / per;
  if (mtl_out != nullptr) *mtl_out = mtl;
}

int64_t w4a16_gemm_tc_workspace(int m, int n, int k) {
  int mt, splits, per;
  tc_plan(m, n, k, &mt, &splits, &per);
  return splits > 1 ? (int64_t)splits * m * n * 4 : 0;
}

// y == nullptr: leave the fp32 partial sums of all `*splits_out` K splits in the workspace
// (after its 16 KB head) for a fused consumer; no bias is applied.
int w4a16_gemm_tc(const half* x, const quic_w4_t& w, half* y, int m, float* workspace, cudaStream_t st,
                  int* splits_out) {
  QUIC_REQUIRE(w.n % kTileN == 0 && w.k % kStageK == 0, QUIC_E_SHAPE,
               "w4a16_linear: the tensor path needs N and K multiples of 128");
  QUIC_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w.qw % 16 == 0), QUIC_E_ARG,
               "w4a16_linear: x and the packed weights must be 16-byte aligned");
  QUIC_REQUIRE(((uintptr_t)w.sc % 16 == 0) && ((uintptr_t)w.zp % 16 == 0), QUIC_E_ARG,
               "w4a16_linear: scales and zero points must be 16-byte aligned");
  int mt, splits, per, mtl;
  tc_plan(m, w.n, w.k, &mt, &splits, &per, &mtl);
  QUIC_REQUIRE((splits == 1 && y != nullptr) || workspace != nullptr, QUIC_E_ARG,
               "w4a16_linear: split-K needs a workspace");
  if (splits_out != nullptr) *splits_out = splits;
  GemmArgs a = {};
  a.w = w;
  a.y = y;
  a.counters = reinterpret_cast<int*>(workspace);
  a.part = workspace + kCounterInts;
  QUIC_REQUIRE((m + mt - 1) / mt <= 65535, QUIC_E_LIMIT, "w4a16_linear: too many rows on the tensor path");
  a.m_total = m;
  a.kblocks_per_split = per;
  a.mtl = mtl;
  int rc;
  switch (mt) {
    case 16: rc = run<16>(x, a, splits, st); break;
    case 32: rc = run<32>(x, a, splits, st); break;
    case 64: rc = run<64>(x, a, splits, st); break;
    default: rc = run<128>(x, a, splits, st); break;
  }
  if (rc != QUIC_OK) return rc;
  if (splits > 1 && y != nullptr) {
    const size_t total = (size_t)m * w.n;
    QUIC_CUDA(launch(tc_splitk_finish_kernel, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0, st, true,
                     (const float*)a.part, (const half*)w.bias, y, m, w.n, splits));
  }
  return QUIC_OK;
}

// act[m, N/2] = silu(x . Wgate^T) * (x . Wup^T) for the fused gate|up weight (N = 2 x 4864, gate
// rows first): one GEMM whose epilogue applies SwiGLU, so the [m, N] intermediate never
// exists.  K is never split here (the activation is not linear in the partial sums).
int w4a16_gemm_tc_swiglu(const half* x, const quic_w4_t& w, half* act, int m, cudaStream_t st) {
  QUIC_REQUIRE(w.n % kTileN == 0 && (w.n / 2) % (kTileN / 2) == 0 && w.k % kStageK == 0, QUIC_E_SHAPE,
               "w4a16 gate_up: N must be a multiple of 128 and K of 128");
  QUIC_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w.qw % 16 == 0) && act != nullptr, QUIC_E_ARG,
               "w4a16 gate_up: x and the packed weights must be 16-byte aligned");
  QUIC_REQUIRE(((uintptr_t)w.sc % 16 == 0) && ((uintptr_t)w.zp % 16 == 0), QUIC_E_ARG,
               "w4a16 gate_up: scales and zero points must be 16-byte aligned");
  int mt, splits, per, mtl;
  tc_plan(m, w.n, w.k, &mt, &splits, &per, &mtl);
  GemmArgs a = {};
  a.w = w;
  a.y = act;
  a.m_total = m;
  a.kblocks_per_split = w.k / kStageK;
  a.mtl = mtl;
  a.fuse_swiglu = 1;
  QUIC_REQUIRE((m + mt - 1) / mt <= 65535, QUIC_E_LIMIT, "w4a16 gate_up: too many rows on the tensor path");
  switch (mt) {
    case 16: return run<16>(x, a, 1, st);
    case 32: return run<32>(x, a, 1, st);
    case 64: return run<64>(x, a, 1, st);
    default: return run<128>(x, a, 1, st);
  }
}

}  // namespace quic

namespace quic {
namespace {
__global__ void tc_status_take_kernel(int* out) {
  out[0] = atomicExch(&g_tc_status[0], 0);
  out[1] = atomicExch(&g_tc_status[1], 0);
}
struct StatusHost {
  int* words[16] = {};   // device address of g_tc_status per device
  int* pinned = nullptr;  // two page-locked ints the status travels through
};
StatusHost g_status_host;
}  // namespace

// Device address of the error words (index 1 is the tensor lm_head's).  Looks the symbol up on
// first use per device: call it once outside any stream capture.
int* tc_status_words() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
  if (g_status_host.words[dev] == nullptr)
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&g_status_host.words[dev]), g_tc_status) != cudaSuccess)
      return nullptr;
  return g_status_host.words[dev];
}

// Enqueues a copy of the error words to page-locked host memory on `st`; tc_status_polled()
// reads them once the stream has been synchronised.  Costs no synchronisation of its own.
int tc_status_poll_async(cudaStream_t st) {
  int* words = tc_status_words();
  if (words == nullptr) return QUIC_OK;
  if (g_status_host.pinned == nullptr)
    QUIC_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&g_status_host.pinned), 2 * sizeof(int), cudaHostAllocDefault));
  QUIC_CUDA(cudaMemcpyAsync(g_status_host.pinned, words, 2 * sizeof(int), cudaMemcpyDeviceToHost, st));
  return QUIC_OK;
}
// After the stream of tc_status_poll_async is idle: 0, or the first non-zero word, which is then
// taken (exchanged with zero on the device, so a word set meanwhile is not lost).
int tc_status_polled(cudaStream_t st) {
  if (g_status_host.pinned == nullptr) return 0;
  const int v = g_status_host.pinned[0] ? g_status_host.pinned[0] : g_status_host.pinned[1];
  if (v == 0) return 0;
  tc_status_take_kernel<<<1, 1, 0, st>>>(g_status_host.pinned);  // page-locked memory is device-accessible (UVA)
  cudaStreamSynchronize(st);
  return v;
}
}  // namespace quic

// Error word of the tensor path: 0, or (code << 16 | block) of the first bounded wait that gave
// up since the last call (code 1: a weight tile never landed, 2: a ring stage never drained,
// 3: operands or the accumulation never completed; bit 15 marks the tensor lm_head).  The word
// is exchanged with zero on the device.  Synchronises the device.
extern "C" int quic_w4a16_tensor_status(void) {
  if (quic::tc_status_words() == nullptr) return -1;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (quic::tc_status_poll_async(nullptr) != QUIC_OK) return -1;
  if (cudaStreamSynchronize(nullptr) != cudaSuccess) return -1;
  return quic::tc_status_polled(nullptr);
}

// Test hook for the bounded waits of the tcgen05 GEMM: launches that follow probe at most
// `spin_limit` times per wait (0 restores the default) and never request the packed weight
// tile of k block `skip_kblock` (128 k per block; -1: none), so the waits for it run out, the
// CTA's roles leave their loops, the error word is set and the kernel returns with its tensor
// memory released.  Nothing faults and nothing waits without a bound.
extern "C" void quic_w4a16_tensor_test_hook(uint32_t spin_limit, int32_t skip_kblock) {
  quic::g_spin_limit = spin_limit ? spin_limit : quic::kSpinLimit;
  quic::g_skip_kblock = skip_kblock;
}
