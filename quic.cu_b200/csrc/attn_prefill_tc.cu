// Causal prefill attention on tcgen05 with TMA-staged tiles (GQA 14:2, head_dim 64): the
// throughput form of attn_prefill.cu for prompts of 128 tokens and more.
//
// Replaces the reference's prefill attention (kernels/flash_attn_prefill_pytorch.py:10 = torch
// SDPA with a causal + left-pad mask; kernels/cuda/flash_attn_prefill.cu:87, wgmma + TMA on
// Hopper).  Same mathematics as attn_prefill.cu: fp32 online softmax over the keys
// 0 .. position of each query row; the probabilities multiply V as fp16 and are summed in fp32.
//
// One CTA owns 128 query rows of one (sequence, query head) and walks the key tiles of 64
// tokens its rows may see.  Per tile:
//   S = Q K^T      tcgen05.mma, A = Q tile (128 x 64, loaded once), B = K tile (64 x 64), both
//                  K-major in the 128-byte swizzle TMA writes; S (128 x 64 fp32) in tensor memory;
//   softmax        eight warps; a thread owns one query row (TMEM lane = row) and half of the
//                  tile's keys: tcgen05.ld its 32 scores, mask, row maximum (exchanged with the warp
//                  that holds the other half), P = exp2(..) rounded to fp16 and stored as the
//                  swizzled A operand of the second product;
//   O_tile = P V   tcgen05.mma, B = V^T.  V sits token-major in the cache, so the same warps
//                  transpose the 64 x 64 tile in shared memory (ldmatrix.trans / stmatrix, two
//                  instructions each per warp) while the first product runs; O_tile
//                  (128 x 64 fp32) in tensor memory;
//   O = alpha O + O_tile in registers (32 dims per thread), alpha = exp2(m_old - m_new).
// K and V tiles arrive through a two-stage TMA ring (plain cp.async.bulk.tensor, no cluster
// multicast; the tensor maps cover this GPU's own cache planes and query buffer).  P, V^T and
// O_tile are double-buffered, and so is S: the scores run two tiles ahead of the softmax, the
// second product of tile i runs while the softmax warps work on tile i + 1 and is folded into O
// one tile late, so no role waits for the tensor pipe in the steady state; two CTAs share an SM.
//
// Roles: warps 0-7 softmax / transpose / epilogue (two per TMEM lane quarter, each half of a tile's
// keys and half of the output dims), warp 8 TMA producer, warp 9 MMA issuer.
// Every wait is bounded; a wait that runs out sets word 0 of the tensor path's error words
// and the CTA leaves with its tensor memory released.
#include "tc_common.cuh"

namespace quic {
namespace {

constexpr int kQRows = 128;   // query rows per CTA (UMMA M)
constexpr int kKeys = 64;     // keys per tile (UMMA N of the first product, K of the second)
constexpr int kSoftmaxWarps = 8;  // two per TMEM lane quarter: each takes half of a tile's keys and half of the dims
constexpr int kAttThreads = (kSoftmaxWarps + 2) * 32;
constexpr uint32_t kQBytes = kQRows * 128;   // 128 rows x 64 halves
constexpr uint32_t kTileBytes = kKeys * 128;  // 64 rows x 64 halves
// Q | K x2 (ring) | V as loaded x2 (ring) | V^T x2 | P x2 (the second product of tile i may still
// run while tile i + 1 goes through the softmax)
constexpr uint32_t kSmemQ = 0, kSmemK = kQBytes, kSmemVraw = kSmemK + 2 * kTileBytes, kSmemVt = kSmemVraw + 2 * kTileBytes,
                   kSmemP = kSmemVt + 2 * kTileBytes, kSmemTotal = kSmemP + 2 * kQBytes + 1024;
constexpr uint32_t kTmemCols = 256;  // S of even / odd tiles: 0..63 / 64..127, O_tile of even / odd tiles: 128..191 / 192..255

struct PrefillTcArgs {
  const int32_t* seq_start;
  const int32_t* seq_len;
  const int32_t* seq_slot;
  const int32_t* seq_off;  // or nullptr
  half* out;               // [rows][896]
  int32_t rows, s_max, n_slots;
  float scale_log2;        // softmax scale x log2(e)
};

__device__ __forceinline__ uint32_t pack2(float x, float y) {
  const half2 h = __floats2half2_rn(x, y);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ void mbar_arrive_cta(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait by polling (mbarrier.test_wait returns at once; try_wait may suspend the thread for a
// scheduling quantum even when the phase completes a few cycles later): for the softmax warps, whose
// barriers are normally complete, or about to be, when they look.
__device__ __forceinline__ bool mbar_poll(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
// barrier of the two warps that share a TMEM lane quarter (ids 1..4; 0 is the CTA barrier)
__device__ __forceinline__ void pair_sync(int quarter) {
  asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
}
// 2^x, one MUFU instruction (x = -inf gives 0)
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kAttThreads, 2) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q,
                                                                         const __grid_constant__ CUtensorMap tm_k,
                                                                         const __grid_constant__ CUtensorMap tm_v,
                                                                         const PrefillTcArgs a, int* status) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bar_q, bar_full[2], bar_empty[2], bar_s[2], bar_p[2], bar_o[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int fail_s;
  __shared__ float pmax_s[2][2][kQRows];  // [tile parity][key half][row]: a warp's row maxima for its partner
  __shared__ float lsum_s[2][kQRows];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.y, seq = blockIdx.z;
  const int len = a.seq_len[seq];  // (the sequence tables are not written by the kernels before this one)
  const int r0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * kQRows;  // the longest key ranges are launched first
  if (r0 >= len) return;
  const int start = a.seq_start[seq];
  const int off = a.seq_off != nullptr ? max(a.seq_off[seq], 0) : 0;
  const int kv_len = off + len;
  const int slot = a.seq_slot[seq];
  if (slot < 0 || slot >= a.n_slots) return;
  const int kvh = head / (kHeads / kKvHeads);
  const int kv_row0 = (slot * kKvHeads + kvh) * a.s_max;  // first row of the (slot, kv head) in the cache plane
  const int n_tiles = (min(kv_len, off + r0 + kQRows) + kKeys - 1) / kKeys;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));

  if (tid == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    mbar_init(smem_u32(&bar_q), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), kSoftmaxWarps);
    }
    mbar_init(smem_u32(&bar_s[0]), 1);
    mbar_init(smem_u32(&bar_s[1]), 1);
    mbar_init(smem_u32(&bar_p[0]), kSoftmaxWarps);
    mbar_init(smem_u32(&bar_p[1]), kSoftmaxWarps);
    mbar_init(smem_u32(&bar_o[0]), 1);
    mbar_init(smem_u32(&bar_o[1]), 1);
    fail_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_s = tmem_base_s, tmem_o = tmem_base_s + 128u;  // S(i) at tmem_s + 64 (i & 1), O_tile(i) at tmem_o + 64 (i & 1)
  const uint32_t idesc = umma_idesc_f16(kKeys);  // M = 128, N = 64 for both products
  pdl_launch_dependents();
  pdl_wait();  // queries and cache rows come from the kernels before this one

  if (warp == kSoftmaxWarps) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      mbar_expect_tx(smem_u32(&bar_q), kQBytes);
      tma_load_2d(base + kSmemQ, &tm_q, 0, head * a.rows + start + r0, smem_u32(&bar_q));
      for (int i = 0; i < n_tiles; ++i) {
        const int st = i & 1;
        if (i >= 2 && !mbar_wait(smem_u32(&bar_empty[st]), ((i >> 1) - 1) & 1)) {
          fail_s = 2;
          break;
        }
        const uint32_t full = smem_u32(&bar_full[st]);
        mbar_expect_tx(full, 2 * kTileBytes);
        tma_load_2d(base + kSmemK + st * kTileBytes, &tm_k, 0, kv_row0 + i * kKeys, full);
        tma_load_2d(base + kSmemVraw + st * kTileBytes, &tm_v, 0, kv_row0 + i * kKeys, full);
      }
    }
  } else if (warp == kSoftmaxWarps + 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // The scores run two tiles ahead of the softmax (two S buffers): S(i + 2) is issued behind the
      // second product of tile i, so the softmax warps never wait for the first product.
      auto scores = [&](int i) {
        const int st = i & 1;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16(tmem_s + 64u * st, umma_desc_sw128(base + kSmemQ + k * 32),
                   umma_desc_sw128(base + kSmemK + st * kTileBytes + k * 32), idesc, k > 0 ? 1u : 0u);
        umma_commit(smem_u32(&bar_s[st]));
      };
      bool ok = mbar_wait(smem_u32(&bar_q), 0);
      for (int i = 0; ok && i < 2 && i < n_tiles; ++i) {
        ok = mbar_wait(smem_u32(&bar_full[i]), 0);
        if (ok) {
          tc_fence_after();
          scores(i);
        }
      }
      for (int i = 0; ok && i < n_tiles; ++i) {
        // P(i) and V^T(i) are in shared memory, S(i) and O_tile(i - 2) have been read
        // (one barrier per tile parity: with the scores two tiles ahead a fast pair of warps can be a
        // whole tile in front of a slow one, and its arrival for tile i + 1 must not count for tile i)
        if (!mbar_wait(smem_u32(&bar_p[i & 1]), (i >> 1) & 1)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const int buf = i & 1;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16(tmem_o + 64u * buf, umma_desc_sw128(base + kSmemP + buf * kQBytes + k * 32),
                   umma_desc_sw128(base + kSmemVt + buf * kTileBytes + k * 32), idesc, k > 0 ? 1u : 0u);
        umma_commit(smem_u32(&bar_o[buf]));
        if (i + 2 < n_tiles) {  // K(i + 2) has replaced K(i) in the ring
          if (!mbar_wait(smem_u32(&bar_full[buf]), ((i + 2) >> 1) & 1)) {
            ok = false;
            break;
          }
          tc_fence_after();
          scores(i + 2);
        }
      }
      if (!ok) fail_s = 3;
    }
  } else {
    // ---------------- softmax, V transpose, epilogue ----------------
    // Warp w: TMEM lane quarter w & 3 (query rows 32 (w & 3) ..), half w >> 2 of every tile's 64 keys
    // and of the 64 output dims.  The two warps of a quarter exchange their row maxima through shared
    // memory once per tile.  No warp leaves the loop early: a wait that ran out only stops further
    // waiting, so the pair barriers always match.
    const int quarter = warp & 3, hf = warp >> 2;
    const int row = 32 * quarter + lane;       // TMEM lane
    const int pos = off + r0 + row;            // position of the row in its sequence
    const uint32_t lane_addr = ((uint32_t)(32 * quarter) << 16) + 32u * hf;
    float m_run = -INFINITY, l_run = 0.f;
    float o[32];
#pragma unroll
    for (int d = 0; d < 32; ++d) o[d] = 0.f;
    bool ok = true;
    float alpha_prev = 0.f;  // rescale that goes with O_tile(i - 1), picked up one tile later
    for (int i = 0; i < n_tiles; ++i) {
      const int st = i & 1, t0 = i * kKeys;
      // ---- V(i) -> V^T as the swizzled B operand
      if (ok) ok = mbar_poll(smem_u32(&bar_full[st]), (i >> 1) & 1);
      {
        // 8 x 8 blocks through ldmatrix.trans / stmatrix: block (tb, db) = tokens 8 tb.., dims 8 db..
        // of the tile as loaded ([64 tokens][64 dims], 128-byte rows, swizzled: the eight rows of a
        // block sit in eight different bank groups) becomes the 16-byte chunk tb of rows
        // 8 db .. 8 db + 7 of V^T.  Warp w moves the eight blocks with db = w: two instructions of
        // four blocks each (lanes 8 m .. 8 m + 7 address the rows of block m).
        const uint32_t vraw = base + kSmemVraw + st * kTileBytes, vt = base + kSmemVt + st * kTileBytes;
        const int m = lane >> 3, r = lane & 7;
#pragma unroll
        for (int it = 0; it < 2; ++it) {
          const int tb = 4 * it + m, db = warp;
          uint32_t x0, x1, x2, x3;
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3)
                       : "r"(vraw + sw128_offset(8 * tb + r, db)));
          asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1,%2,%3,%4};" ::"r"(
                           vt + sw128_offset(8 * db + r, tb)),
                       "r"(x0), "r"(x1), "r"(x2), "r"(x3)
                       : "memory");
        }
      }
      // ---- the row's scores for this warp's 32 keys
      if (ok) ok = mbar_poll(smem_u32(&bar_s[st]), (i >> 1) & 1);
      tc_fence_after();
      __syncwarp();  // every lane of the warp has finished its share of the transpose
      if (lane == 0) mbar_arrive_cta(smem_u32(&bar_empty[st]));  // K(i) has been multiplied, V(i) transposed
      const int t_hi = min(pos, kv_len - 1) - t0 - 32 * hf;  // this warp's columns 0 .. t_hi are visible to the row
      // a tile wholly below the diagonal of all 128 rows needs no mask (CTA-uniform)
      const bool unmasked = t0 + kKeys - 1 <= min(off + r0, kv_len - 1);
      float s[32];
      tmem_ld32(tmem_s + 64u * st + lane_addr, s);
      tc_fence_before();  // the loads of S precede the next product into the same columns
      if (!unmasked) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j > t_hi) s[j] = -INFINITY;
      }
      float mx[4];  // independent chains instead of one of 32 dependent maxima
#pragma unroll
      for (int j = 0; j < 4; ++j) mx[j] = s[j];
#pragma unroll
      for (int j = 4; j < 32; ++j) mx[j & 3] = fmaxf(mx[j & 3], s[j]);
      float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      pmax_s[i & 1][hf][row] = mt;
      pair_sync(quarter);
      mt = fmaxf(mt, pmax_s[i & 1][hf ^ 1][row]);
      const float m_new = fmaxf(m_run, mt * a.scale_log2);  // (the scale is positive)
      const float alpha = ex2(m_run - m_new);  // 0 on the first tile (m_run = -inf)
      // m_new is finite from the first tile on: every row sees key 0
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float p0 = ex2(fmaf(s[8 * c + 2 * j], a.scale_log2, -m_new));  // 2^-inf = 0 for masked keys
          const float p1 = ex2(fmaf(s[8 * c + 2 * j + 1], a.scale_log2, -m_new));
          l4[j] += p0 + p1;
          w[j] = pack2(p0, p1);
        }
        *reinterpret_cast<uint4*>(gen + kSmemP + st * kQBytes + sw128_offset(row, 4 * hf + c)) =
            make_uint4(w[0], w[1], w[2], w[3]);
      }
      l_run = l_run * alpha + ((l4[0] + l4[1]) + (l4[2] + l4[3]));  // this warp's keys only; halves added at the end
      m_run = m_new;
      fence_proxy_async();  // P and V^T (generic-proxy stores) -> visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(smem_u32(&bar_p[st]));
      // ---- O = alpha O + P V of the PREVIOUS tile: its product ran while this tile's softmax did
      if (i > 0) {
        if (ok) ok = mbar_poll(smem_u32(&bar_o[(i - 1) & 1]), ((i - 1) >> 1) & 1);
        tc_fence_after();
        {
          float v[32];
          tmem_ld32(tmem_o + 64u * ((i - 1) & 1) + lane_addr, v);
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = fmaf(o[j], alpha_prev, v[j]);
        }
        tc_fence_before();
      }
      alpha_prev = alpha;
    }
    {  // the last tile's product
      const int i = n_tiles - 1;
      if (ok) ok = mbar_poll(smem_u32(&bar_o[i & 1]), (i >> 1) & 1);
      tc_fence_after();
      float v[32];
      tmem_ld32(tmem_o + 64u * (i & 1) + lane_addr, v);
#pragma unroll
      for (int j = 0; j < 32; ++j) o[j] = fmaf(o[j], alpha_prev, v[j]);
      tc_fence_before();
    }
    lsum_s[hf][row] = l_run;
    pair_sync(quarter);
    l_run += lsum_s[hf ^ 1][row];
    ok = ok && !fail_s;
    if (!ok && lane == 0) atomicCAS(status, 0, ((fail_s ? fail_s : 1) << 16) | 0x2000 | ((int)blockIdx.x & 0x1fff));
    if (ok && r0 + row < len) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      half* op = a.out + (size_t)(start + r0 + row) * kHidden + head * kHeadDim + 32 * hf;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint4 u;
        u.x = pack2(o[8 * c + 0] * inv, o[8 * c + 1] * inv);
        u.y = pack2(o[8 * c + 2] * inv, o[8 * c + 3] * inv);
        u.z = pack2(o[8 * c + 4] * inv, o[8 * c + 5] * inv);
        u.w = pack2(o[8 * c + 6] * inv, o[8 * c + 7] * inv);
        reinterpret_cast<uint4*>(op)[c] = u;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_s), "r"(kTmemCols) : "memory");
}

}  // namespace

// Whether the tcgen05 form takes this call (otherwise attn_prefill.cu's mma.sync kernels do).
bool attn_prefill_tc_supported(int n_seq, int max_len, int rows, int s_max, int n_slots) {
  return max_len >= kQRows && (int64_t)n_slots * kKvHeads * s_max < (1ll << 31) && (int64_t)kHeads * rows < (1ll << 31);
}

int attn_prefill_tc_launch(const void* q, const void* kcache, const void* vcache, const int32_t* seq_start,
                           const int32_t* seq_len, const int32_t* seq_slot, const int32_t* seq_off, int32_t n_seq,
                           int32_t max_len, int32_t rows, int32_t s_max, int32_t n_slots, float scale, void* out,
                           cudaStream_t stream, bool pdl) {
  CUtensorMap tm_q, tm_k, tm_v;
  int rc = make_map(&tm_q, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, q, (uint64_t)kHeads * rows, kHeadDim, kQRows, kHeadDim,
                    CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != QUIC_OK) return rc;
  const uint64_t kv_rows = (uint64_t)n_slots * kKvHeads * s_max;
  rc = make_map(&tm_k, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, kcache, kv_rows, kHeadDim, kKeys, kHeadDim,
                CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != QUIC_OK) return rc;
  rc = make_map(&tm_v, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, vcache, kv_rows, kHeadDim, kKeys, kHeadDim,
                CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != QUIC_OK) return rc;
  int* status = tc_status_words();
  QUIC_REQUIRE(status != nullptr, QUIC_E_CUDA, "attn_prefill: no address for the tensor path's error words");
  PrefillTcArgs a = {};
  a.seq_start = seq_start;
  a.seq_len = seq_len;
  a.seq_slot = seq_slot;
  a.seq_off = seq_off;
  a.out = (half*)out;
  a.rows = rows;
  a.s_max = s_max;
  a.n_slots = n_slots;
  a.scale_log2 = (scale > 0.f ? scale : 0.125f) * 1.4426950408889634f;
  QUIC_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTotal));
  dim3 grid((max_len + kQRows - 1) / kQRows, kHeads, n_seq);
  QUIC_CUDA(launch(attn_prefill_tc_kernel, grid, dim3(kAttThreads), kSmemTotal, stream, pdl, tm_q, tm_k, tm_v, a, status));
  return QUIC_OK;
}

}  // namespace quic
