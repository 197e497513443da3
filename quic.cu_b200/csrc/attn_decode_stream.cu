// GQA decode attention for many rows (the tensor-core step beyond 20 rows): ONE CTA per
// (row, KV head) streams that head's cached keys and values through a ring of shared-memory
// stages filled by TMA (64-token tiles, 128-byte swizzle), six warps take the tiles in turn
// -- the 64-token tile arithmetic of attn_warp.cuh on mma.sync, each warp keeping a running
// softmax over its tiles -- and meet once in shared memory.  No partial results in global
// memory, no counters, no second pass, and nothing is read beyond a row's own length.
//
// Why: with one-warp CTAs (attn_decode_warp_kernel) every warp requests its 16 KB tile with 32
// loads per lane and then waits for it; at 64 rows of 200..1500 tokens that form reads 1.8 x
// the algorithmic bytes (tiles beyond a row's length are fetched too), reaches a quarter of the
// HBM bandwidth and takes 25 us per layer (12 us here).  Here a single thread keeps kStreamStages x
// 16 KB of bulk copies in flight per SM and the copies cost the warps no instructions.  Measured
// per 64-row step of 200..1500 tokens: 1266 us with one-warp CTAs, 1022 with four warps and eight
// stages, 1015 with six warps and twelve stages, 973 with the QKV finish below.
//
// Inside the decode chain (a.prefetch) the producer requests, BEFORE the dependency wait, the
// tiles that hold only tokens of earlier steps (up to the ring's depth): those rows are complete
// once the step counter shows the current step.  The counter is read (acquire) before the
// requests and again after the wait; if it moved, the previous step was still finishing when
// the tiles were requested, and they are requested again (a second phase of the same stages'
// barriers, which their consumers then wait for).  The tile of the row that the preceding
// kernel appends is never requested early.
//
// With `fin.part` (or `fin.qkv`, a finished fp16 output) set the CTA first finishes the fused QKV linear for its row and KV head, which a
// separate kernel (qkv_post_kernel) would otherwise do between the GEMM and the attention: the
// compute warps sum the split-K partial sums of their seven q heads, their k head and their v head,
// add the bias with the GEMM epilogue's roundings, rotate q and k (rope.forward of the reference,
// kernels/cuda/rope.cu), keep q in shared memory for the fragments, append k and v to the cache for
// later steps, and the warp that owns the row's last tile writes the new k and v into that tile in
// shared memory once TMA has landed it -- whatever TMA read at that position is overwritten.
//
// Same mathematics as fad_decode_kernel + fad_combine_kernel of the reference
// (kernels/cuda/flash_attn_decode.cu:12,104): fp32 softmax over the tokens [start_b, end_b) of
// each row, rows without tokens give zeros (:118-121).
#include "attn_warp.cuh"
#include "decode_kernels.cuh"
#include "tc_common.cuh"

namespace quic {
namespace {

constexpr int kGroupHeads = kHeads / kKvHeads;  // 7
constexpr int kStreamWarps = 6;                  // compute warps; the next warp is the producer
constexpr int kStreamStages = 12;                // ring depth: 192 KB of copies in flight per SM
// Tile i lives in stage i % kStreamStages and belongs to warp i % kStreamWarps.  The depth must be
// a multiple of the warp count: then every stage is always consumed by the same warp, in order,
// and a parity wait can never be answered by the phase of two uses earlier.  (With 8 warps and 12
// stages, stage 0 holds tiles 0, 12, 24 of warps 0, 4, 0: warp 0 could find the parity of tile 24
// already 'complete' -- it is tile 0's -- while tile 12 was still being consumed.)
static_assert(kStreamStages % kStreamWarps == 0, "every stage must belong to one warp");
constexpr uint32_t kTileBytes = kWarpChunk * kHeadDim * 2;  // 8 KB: 64 tokens x 128 bytes
constexpr uint32_t kStageBytes = 2 * kTileBytes;            // K tile, V tile
constexpr size_t kStreamSmem = (size_t)kStreamStages * kStageBytes + 1024;

__device__ __forceinline__ void mbar_arrive_local(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// The fragments of warp_tile_request, from a swizzled tile pair in shared memory (conflict-free:
// a quarter warp reads eight different 16-byte chunks of the 128-byte bank cycle).
__device__ __forceinline__ void warp_tile_from_smem(WarpTile& t, uint32_t k_s, uint32_t v_s, int g, int c) {
#pragma unroll
  for (int nb = 0; nb < 8; ++nb) {
    const int row = 8 * nb + g;
    t.kr[nb][0] = lds128(k_s + sw128_offset(row, 2 * c));
    t.kr[nb][1] = lds128(k_s + sw128_offset(row, 2 * c + 1));
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int row = 16 * j + 2 * c + (r & 1) + 8 * (r >> 1);
      t.vr[j][r] = lds128(v_s + sw128_offset(row, g));
    }
  }
}

__global__ void __launch_bounds__((kStreamWarps + 1) * 32, 1)
    attn_decode_stream_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                              const AttnArgs a, const QkvFinish fin, int n_slots, int s_max, int* status,
                              int force_reload, int skip_tile0, uint32_t spin_limit) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStreamStages];   // a stage's two tiles landed
  __shared__ __align__(8) uint64_t bar_empty[kStreamStages];  // its consumer warp holds them in registers
  __shared__ float m_s[kStreamWarps][kGroupHeads];
  __shared__ float l_s[kStreamWarps][kGroupHeads];
  __shared__ __align__(16) float o_s[kStreamWarps][kGroupHeads][kHeadDim];
  __shared__ int fail_s, pre_s, epoch_s;
  __shared__ __align__(16) half q_s[kGroupHeads][kHeadDim];  // finished q heads (fin.part set)
  __shared__ __align__(16) half kn_s[kHeadDim], vn_s[kHeadDim];  // this step's k and v of the KV head

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int kvh = blockIdx.x, b = blockIdx.y;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  if (tid == 0) {
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    for (int s = 0; s < kStreamStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    fail_s = 0;
    pre_s = 0;
    epoch_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_trigger_early();
  if (warp == kStreamWarps && lane == 0 && a.prefetch != 0 && a.epoch != nullptr && a.pos != nullptr) {
    const int e0 = ld_acquire_s32(a.epoch);
    const int slot0 = a.rows[b];  // (the row -> slot map is not written inside the chain)
    const int p0 = min(__ldcg(a.pos + slot0), a.s_cap);  // tokens below p0 were appended by earlier steps
    const int pre = min(p0 > 0 ? p0 / kWarpChunk : 0, kStreamStages);
    const int row0p = (slot0 * kKvHeads + kvh) * s_max;
    for (int i = skip_tile0 ? 1 : 0; i < pre; ++i) {  // (test hook: the wait for tile 0 runs out)
      const uint32_t full = smem_u32(&bar_full[i]), dst = base + i * kStageBytes;
      mbar_expect_tx(full, kStageBytes);
      tma_load_2d(dst, &tm_k, 0, row0p + i * kWarpChunk, full);
      tma_load_2d(dst + kTileBytes, &tm_v, 0, row0p + i * kWarpChunk, full);
    }
    pre_s = pre;
    epoch_s = e0;
  }
  pdl_wait();  // the row appended by the preceding kernel and the positions are complete
  __syncthreads();
  const int pre = pre_s;  // tiles requested before the wait (they start at token 0: positions mode)
  const bool stale = pre > 0 && (__ldcg(a.epoch) != epoch_s || force_reload != 0);

  int slot = b, t_begin = 0, t_end = a.s_cap;
  int p_new = -1;  // position of this step's token (positions mode)
  if (a.pos != nullptr) {
    slot = a.rows[b];
    p_new = __ldcg(a.pos + slot);
    t_end = p_new + 1;
  } else {
    if (a.start != nullptr) t_begin = a.start[b];
    if (a.end != nullptr) t_end = a.end[b];
  }
  if (t_end > a.s_cap) t_end = a.s_cap;
  if (t_begin < 0) t_begin = 0;
  const int tile0 = t_begin / kWarpChunk;
  const int n_tiles = t_end > t_begin ? (t_end + kWarpChunk - 1) / kWarpChunk - tile0 : 0;
  const int row0 = (slot * kKvHeads + kvh) * s_max;  // first cache row of this (slot, KV head)

  float m = -INFINITY, l = 0.f, o[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

  const bool finish = fin.part != nullptr || fin.qkv != nullptr;
  if (finish && warp < kStreamWarps) {
    // thread -> (head of the CTA: 7 q, k, v; rotation pair): stored columns (2 pair, 2 pair + 1) are dims (pair, pair + 32)
    const bool slot_ok = slot >= 0 && slot < n_slots;
    const int p = slot_ok ? p_new : 0;
    const int pp = p < fin.max_pos ? (p < 0 ? 0 : p) : fin.max_pos - 1;
    for (int idx = tid; idx < (kGroupHeads + 2) * 32; idx += kStreamWarps * 32) {
      const int hl = idx >> 5, pair = idx & 31;
      const int head = hl < kGroupHeads ? kvh * kGroupHeads + hl : (hl == kGroupHeads ? kHeads + kvh : kHeads + kKvHeads + kvh);
      const int col = head * kHeadDim + 2 * pair;
      float x, y;
      if (fin.qkv != nullptr) {  // the dense GEMM's own output, bias included
        const float2 v = __half22float2(*reinterpret_cast<const half2*>(fin.qkv + (size_t)b * kQkvN + col));
        x = v.x;
        y = v.y;
      } else {
      float2 acc = make_float2(0.f, 0.f);
      for (int s0 = 0; s0 < fin.splits; s0 += 8) {  // eight partial sums in flight
        float2 ps[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          ps[j] = s0 + j < fin.splits
                      ? __ldcg(reinterpret_cast<const float2*>(fin.part + ((size_t)(s0 + j) * gridDim.y + b) * kQkvN + col))
                      : make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc.x += ps[j].x;
          acc.y += ps[j].y;
        }
      }
      const float2 bb = __half22float2(*reinterpret_cast<const half2*>(fin.bias + col));
      x = __half2float(__float2half_rn(__half2float(__float2half_rn(acc.x)) + bb.x));
      y = __half2float(__float2half_rn(__half2float(__float2half_rn(acc.y)) + bb.y));
      }
      float lo = x, hi = y;
      if (hl <= kGroupHeads) {  // q and k are rotated
        const float cs = __half2float(fin.cos_t[(size_t)pp * 32 + pair]), sn = __half2float(fin.sin_t[(size_t)pp * 32 + pair]);
        lo = x * cs - y * sn;
        hi = x * sn + y * cs;
      }
      const half hlo = __float2half_rn(lo), hhi = __float2half_rn(hi);
      if (hl < kGroupHeads) {
        q_s[hl][pair] = hlo;
        q_s[hl][pair + 32] = hhi;
      } else {
        half* mine = hl == kGroupHeads ? kn_s : vn_s;
        mine[pair] = hlo;
        mine[pair + 32] = hhi;
        if (slot_ok && p >= 0 && p < s_max) {  // for the steps to come
          half* dst = const_cast<half*>(hl == kGroupHeads ? a.k : a.v) + ((size_t)row0 + p) * kHeadDim;
          dst[pair] = hlo;
          dst[pair + 32] = hhi;
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kStreamWarps * 32) : "memory");  // the compute warps only
  }

  if (warp == kStreamWarps) {
    // ---------------- producer: one thread keeps the ring full ----------------
    if (lane == 0) {
      int repeated = 0, issued = pre;  // early copies fetched again; tiles requested so far
      if (stale) {  // wait for the early copies to land, then fetch the same tiles again
        for (int i = 0; i < pre; ++i, ++repeated) {
          const uint32_t full = smem_u32(&bar_full[i]), dst = base + i * kStageBytes;
          if (!mbar_wait(full, 0, spin_limit)) {
            fail_s = 1;
            break;
          }
          mbar_expect_tx(full, kStageBytes);
          tma_load_2d(dst, &tm_k, 0, row0 + i * kWarpChunk, full);
          tma_load_2d(dst + kTileBytes, &tm_v, 0, row0 + i * kWarpChunk, full);
        }
      }
      for (int i = pre; i < n_tiles && fail_s == 0; ++i, ++issued) {
        const int s = i % kStreamStages;
        if (i >= kStreamStages && !mbar_wait(smem_u32(&bar_empty[s]), ((i / kStreamStages) - 1) & 1, spin_limit)) {
          fail_s = 1;
          break;
        }
        if (i == 0 && skip_tile0) continue;  // (test hook)
        const uint32_t full = smem_u32(&bar_full[s]), dst = base + s * kStageBytes;
        const int row = row0 + (tile0 + i) * kWarpChunk;  // rows past the end of the cache read as zero
        mbar_expect_tx(full, kStageBytes);
        tma_load_2d(dst, &tm_k, 0, row, full);
        tma_load_2d(dst + kTileBytes, &tm_v, 0, row, full);
      }
      // No copy may still be on its way into this CTA's shared memory when the CTA ends, whatever
      // became of its consumer: wait (with the usual bound) for the last copy into every stage.
      // In the normal course the consumers needed these phases anyway.
      for (int i = issued > kStreamStages ? issued - kStreamStages : 0; i < issued; ++i) {
        const int s = i % kStreamStages;
        const int phase = i / kStreamStages + ((i < pre ? i < repeated : (stale && s < pre)) ? 1 : 0);
        if (!mbar_wait(smem_u32(&bar_full[s]), phase & 1, spin_limit)) fail_s = 1;
      }
    }
  } else if (n_tiles > 0) {
    // ---------------- compute warps: tile i belongs to warp i % kStreamWarps ----------------
    uint32_t qa0[4], qa2[4];
    if (finish) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        qa0[ks] = qa2[ks] = 0u;
        if (g < kGroupHeads) {
          const uint2 u = *reinterpret_cast<const uint2*>(&q_s[g][16 * c + 4 * ks]);
          qa0[ks] = u.x;
          qa2[ks] = u.y;
        }
      }
    } else {
      warp_q_fragments(qa0, qa2, a.q + ((size_t)b * kHeads + kvh * kGroupHeads) * kHeadDim, g, c);
    }
    for (int i = warp; i < n_tiles; i += kStreamWarps) {
      const int s = i % kStreamStages;
      // (a stage whose early copy was repeated is one phase ahead for the rest of the kernel)
      const int shift = (stale && s < pre) ? 1 : 0;
      bool ok = mbar_wait(smem_u32(&bar_full[s]), ((i / kStreamStages) + shift) & 1, spin_limit);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) fail_s = 2;
        break;
      }
      const int t0 = (tile0 + i) * kWarpChunk;
      if (finish && p_new >= t0 && p_new < t0 + kWarpChunk && p_new < t_end) {
        // this step's k and v take their row of the tile (16 chunks of 16 bytes: lanes 0-7 k, 8-15 v)
        if (lane < 16) {
          const int chunk = lane & 7;
          const uint32_t dst = base + s * kStageBytes + (lane < 8 ? 0u : kTileBytes) + sw128_offset(p_new - t0, chunk);
          const uint4 val = *reinterpret_cast<const uint4*>((lane < 8 ? kn_s : vn_s) + 8 * chunk);
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(val.x), "r"(val.y), "r"(val.z), "r"(val.w)
                       : "memory");
        }
        __syncwarp();
      }
      WarpTile tile;
      warp_tile_from_smem(tile, base + s * kStageBytes, base + s * kStageBytes + kTileBytes, g, c);
      __syncwarp();
      if (lane == 0) mbar_arrive_local(smem_u32(&bar_empty[s]));  // the stage may be refilled
      float m1, l1, o1[8][4];
      warp_tile_attend(tile, qa0, qa2, t0, max(t_begin, t0), min(t_end, t0 + kWarpChunk), a.scale, c, m1, l1, o1);
      // running softmax over this warp's tiles (m, l are equal in the four lanes of a head)
      const float mx = fmaxf(m, m1);
      if (mx != -INFINITY) {
        const float e0 = (m == -INFINITY) ? 0.f : __expf(m - mx);
        const float e1 = (m1 == -INFINITY) ? 0.f : __expf(m1 - mx);
        l = e0 * l + e1 * l1;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j][0] = e0 * o[j][0] + e1 * o1[j][0];
          o[j][1] = e0 * o[j][1] + e1 * o1[j][1];
        }
        m = mx;
      }
    }
  }
  if (warp < kStreamWarps && g < kGroupHeads) {
    // C columns 2c, 2c+1 of mma j are dims 16c + j and 16c + 8 + j of head g
    float4* op = reinterpret_cast<float4*>(&o_s[warp][g][16 * c]);
    op[0] = make_float4(o[0][0], o[1][0], o[2][0], o[3][0]);
    op[1] = make_float4(o[4][0], o[5][0], o[6][0], o[7][0]);
    op[2] = make_float4(o[0][1], o[1][1], o[2][1], o[3][1]);
    op[3] = make_float4(o[4][1], o[5][1], o[6][1], o[7][1]);
    if (c == 0) {
      m_s[warp][g] = m;
      l_s[warp][g] = l;
    }
  }
  __syncthreads();
  if (fail_s != 0) {  // a bounded wait gave up: say so, leave the row's output as it is
    if (tid == 0) atomicCAS(status, 0, ((4 + fail_s) << 16) | 0x4000 | ((int)blockIdx.y & 0x3fff));
    return;
  }
  // the warps' results -> the row's heads; thread -> (head, pair of dims), 224 of them
  for (int idx = tid; idx < kGroupHeads * 32; idx += (kStreamWarps + 1) * 32) {
    const int h = idx >> 5, d2 = idx & 31;
    float mx = -INFINITY, den = 0.f;
    float2 num = make_float2(0.f, 0.f);
#pragma unroll
    for (int w = 0; w < kStreamWarps; ++w) mx = fmaxf(mx, m_s[w][h]);
    if (mx != -INFINITY) {
#pragma unroll
      for (int w = 0; w < kStreamWarps; ++w) {
        const float e = (m_s[w][h] == -INFINITY) ? 0.f : __expf(m_s[w][h] - mx);
        const float2 v = *reinterpret_cast<const float2*>(&o_s[w][h][2 * d2]);
        den = fmaf(e, l_s[w][h], den);
        num.x = fmaf(e, v.x, num.x);
        num.y = fmaf(e, v.y, num.y);
      }
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    *reinterpret_cast<half2*>(a.out + ((size_t)b * kHeads + kvh * kGroupHeads + h) * kHeadDim + 2 * d2) =
        __floats2half2_rn(num.x * inv, num.y * inv);
  }
}

}  // namespace

// The cache planes must be the decode step's: [n_slots][2][s_max][64] fp16, 16-byte aligned.
// a.s_cap bounds the tokens of a row; `status`: error word of the bounded waits.
int g_stream_hook = 0;  // quic_attn_stream_test_hook: 1 repeat the early requests, 2 never request tile 0

int launch_attn_stream(const AttnArgs& a, const QkvFinish* fuse, int batch, int n_slots, int s_max, int* status,
                       cudaStream_t stream, bool pdl) {
  QUIC_REQUIRE(a.stride_h == (int64_t)s_max * kHeadDim && a.stride_b == (int64_t)kKvHeads * s_max * kHeadDim,
               QUIC_E_ARG, "attn_decode_stream: the cache must be [slots][2][s_max][64]");
  QUIC_REQUIRE(status != nullptr && batch >= 1 && batch <= 65535 && n_slots >= 1, QUIC_E_ARG,
               "attn_decode_stream: bad batch, slots or status word");
  QkvFinish fin = {};
  if (fuse != nullptr) {
    QUIC_REQUIRE(((fuse->part && fuse->bias && fuse->splits >= 1) || fuse->qkv) && fuse->cos_t && fuse->sin_t &&
                     fuse->max_pos >= 1 && a.pos != nullptr && a.rows != nullptr,
                 QUIC_E_ARG, "attn_decode_stream: incomplete QKV finish");
    fin = *fuse;
  }
  CUtensorMap tm_k, tm_v;
  const uint64_t rows = (uint64_t)n_slots * kKvHeads * s_max;
  int rc = make_map(&tm_k, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.k, rows, kHeadDim, kWarpChunk, kHeadDim,
                    CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != QUIC_OK) return rc;
  rc = make_map(&tm_v, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.v, rows, kHeadDim, kWarpChunk, kHeadDim,
                CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != QUIC_OK) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    QUIC_CUDA(cudaFuncSetAttribute(attn_decode_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)kStreamSmem));
    attr_set = true;
  }
  QUIC_CUDA(launch(attn_decode_stream_kernel, dim3(kKvHeads, batch), dim3((kStreamWarps + 1) * 32), kStreamSmem, stream,
                   pdl, tm_k, tm_v, a, fin, n_slots, s_max, status, g_stream_hook == 1 ? 1 : 0, g_stream_hook == 2 ? 1 : 0,
                   g_stream_hook == 2 ? 20000u : kSpinLimit));
  return QUIC_OK;
}

}  // namespace quic

// Test hook for the launches (and graph captures) that follow.  1: the kernel treats its early tile
// requests as made too early and repeats them, as it does when the step counter moved between the
// request and the dependency wait.  2: the first tile of every row is never requested and the
// waits probe 20000 times at most, so the wait for that tile runs out, the other roles' waits
// follow, the CTA sets the error word (code 5 or 6, bit 14) and returns; nothing faults.  0: normal.
extern "C" void quic_attn_stream_test_hook(int32_t mode) { quic::g_stream_hook = (mode == 1 || mode == 2) ? mode : 0; }
