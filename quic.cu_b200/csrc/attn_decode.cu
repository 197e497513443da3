// Split-K GQA decode attention over an fp16 K/V cache, head_dim 64, 7 query
// heads per KV head.
//
// Replaces fad_decode_kernel + fad_combine_kernel of the reference
// (kernels/cuda/flash_attn_decode.cu:12,104).  Same mathematics — fp32 online
// softmax over the tokens [start_b, end_b) of each row, rows without tokens
// give zeros (:118-121) — with three kernels for three regimes:
//   * attn_decode_warp_kernel (latency: the decode chain up to 2048 tokens, small problems):
//     ONE WARP per 64 tokens of a (row, kv head), both products on mma.sync.m16n8k16, no
//     shared memory; inside the chain its cache tile is requested before the dependency wait;
//   * attn_decode_mma_kernel (throughput): 4 or 8 warps per CTA walking 32-token tiles with an
//     online softmax, the same mma.sync fragment mappings (attn_warp.cuh), warps merged
//     through shared memory;
//   * attn_decode_kernel (scalar, kept for small stand-alone problems): one token per lane
//     for q.k, all 7 query heads of the group at once.
// Splits go through global fp32 partials; they are merged by the consumer (the o_proj kernel
// of the small-batch chain) or by the CTA that arrives last at a per-(row, kv head) counter,
// which re-arms the counter, so no second kernel and no spin-wait is needed.
#include "decode_kernels.cuh"
#include "attn_warp.cuh"

// Bytes reserved for the arrival counters at the head of the scratch: a fixed 64 KB (8192
// rows) so that a scratch block shared by calls of different batch sizes keeps its counters
// apart from the partials whatever the layout of the previous call was.
static int64_t counter_bytes(int b) {
  const int64_t need = ((int64_t)b * QUIC_KV_HEADS * 4 + 255) / 256 * 256;
  return need > 65536 ? need : 65536;
}


namespace quic {
namespace {

constexpr int kGroupHeads = kHeads / kKvHeads;  // 7

constexpr int kWarps = 8;
constexpr int kTile = 32;

// The same merge for single-warp CTAs and at most 32 splits.  Lane s owns split s for the
// softmax statistics (one coalesced load per head), every lane owns two dims of the output;
// all partial loads of four heads are in flight together, so the merge costs three memory
// round trips whatever the split count.
__device__ __forceinline__ void merge_splits_warp(const AttnArgs& a, int b, int kvh) {
  const int lane = threadIdx.x;
  __threadfence();
  __syncwarp();
  int old = 0;
  if (lane == 0) old = atomicAdd(&a.counters[b * kKvHeads + kvh], 1);
  old = __shfl_sync(0xffffffffu, old, 0);
  if (old != a.splits - 1) return;
  __threadfence();
  const size_t row0 = ((size_t)b * kHeads + kvh * kGroupHeads) * a.splits;
  float e[kGroupHeads], inv[kGroupHeads];
  {
    float ms[kGroupHeads], ls[kGroupHeads];
#pragma unroll
    for (int h = 0; h < kGroupHeads; ++h) {
      const bool in = lane < a.splits;
      ms[h] = in ? __ldcg(a.m_part + row0 + (size_t)h * a.splits + lane) : -INFINITY;
      ls[h] = in ? __ldcg(a.l_part + row0 + (size_t)h * a.splits + lane) : 0.f;
    }
#pragma unroll
    for (int h = 0; h < kGroupHeads; ++h) {
      const float mx = warp_max(ms[h]);
      e[h] = (ms[h] == -INFINITY) ? 0.f : __expf(ms[h] - mx);
      const float den = warp_sum(e[h] * ls[h]);
      inv[h] = den > 0.f ? 1.f / den : 0.f;
    }
  }
  constexpr int kBatchHeads = 4;
#pragma unroll
  for (int h0 = 0; h0 < kGroupHeads; h0 += kBatchHeads) {
    float2 acc[kBatchHeads];
#pragma unroll
    for (int hh = 0; hh < kBatchHeads; ++hh) acc[hh] = make_float2(0.f, 0.f);
    for (int s0 = 0; s0 < a.splits; s0 += 8) {
      float2 v[kBatchHeads][8];
#pragma unroll
      for (int hh = 0; hh < kBatchHeads; ++hh) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const bool in = (h0 + hh < kGroupHeads) && (s0 + j < a.splits);
          v[hh][j] = in ? __ldcg(reinterpret_cast<const float2*>(
                              a.o_part + (row0 + (size_t)(h0 + hh) * a.splits + s0 + j) * kHeadDim) + lane)
                        : make_float2(0.f, 0.f);
        }
      }
#pragma unroll
      for (int hh = 0; hh < kBatchHeads; ++hh) {
        if (h0 + hh >= kGroupHeads) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float w = __shfl_sync(0xffffffffu, e[h0 + hh], (s0 + j) & 31);
          acc[hh].x = fmaf(w, v[hh][j].x, acc[hh].x);
          acc[hh].y = fmaf(w, v[hh][j].y, acc[hh].y);
        }
      }
    }
#pragma unroll
    for (int hh = 0; hh < kBatchHeads; ++hh) {
      if (h0 + hh >= kGroupHeads) continue;
      const int qh = kvh * kGroupHeads + h0 + hh;
      *reinterpret_cast<half2*>(a.out + ((size_t)b * kHeads + qh) * kHeadDim + 2 * lane) =
          __floats2half2_rn(acc[hh].x * inv[h0 + hh], acc[hh].y * inv[h0 + hh]);
    }
  }
  if (lane == 0) a.counters[b * kKvHeads + kvh] = 0;
}

__global__ void __launch_bounds__(kWarps * 32) attn_decode_kernel(const AttnArgs a) {
  __shared__ __align__(16) float q_s[kGroupHeads * kHeadDim];
  __shared__ __align__(16) float p_s[kWarps][kGroupHeads][kTile];
  __shared__ float m_s[kWarps][kGroupHeads];
  __shared__ float l_s[kWarps][kGroupHeads];
  __shared__ __align__(16) float o_s[kWarps][kGroupHeads][kHeadDim];
  __shared__ int last_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;

  // The row -> slot map is not written by any kernel of the decode chain.
  int slot = b;
  if (a.pos != nullptr) slot = a.rows[b];
  pdl_trigger_early();
  pdl_wait();

  const half* kbase = a.k + (size_t)slot * a.stride_b + (size_t)kvh * a.stride_h;
  const half* vbase = a.v + (size_t)slot * a.stride_b + (size_t)kvh * a.stride_h;
  const int vt = lane >> 3;        // token (mod 4) this lane covers in p·V
  const int vd = (lane & 7) * 8;   // first of its 8 dims
  const int last_tok = a.s_cap - 1;

  // One round of global loads: the first K/V tile of this warp is requested
  // before the row's token range is known (its position in the cache is fixed
  // by the split; tokens outside the range are masked later, addresses are
  // clamped into the cache), together with the range itself and q.
  uint4 kr[8], vr[8];
  int t0 = split * a.chunk + warp * kTile;
  {
    const uint4* kp = reinterpret_cast<const uint4*>(kbase + (size_t)min(t0 + lane, last_tok) * kHeadDim);
#pragma unroll
    for (int i = 0; i < 8; ++i) kr[i] = ldg_nc_u128(kp + i);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      vr[i] = ldg_nc_u128(vbase + (size_t)min(t0 + 4 * i + vt, last_tok) * kHeadDim + vd);
  }
  int t_begin = 0, t_end = a.s_cap;
  if (a.pos != nullptr) {
    t_end = __ldcg(a.pos + slot) + 1;
  } else {
    if (a.start != nullptr) t_begin = a.start[b];
    if (a.end != nullptr) t_end = a.end[b];
  }
  for (int i = tid; i < kGroupHeads * kHeadDim; i += kWarps * 32)
    q_s[i] = __half2float(a.q[((size_t)b * kHeads + kvh * kGroupHeads) * kHeadDim + i]) * a.scale;
  if (t_end > a.s_cap) t_end = a.s_cap;
  if (t_begin < 0) t_begin = 0;
  const int c_begin = max(t_begin, split * a.chunk);
  const int c_end = min(t_end, (split + 1) * a.chunk);
  __syncthreads();

  float m_run[kGroupHeads], l_run[kGroupHeads];
  float o[kGroupHeads][8];
#pragma unroll
  for (int h = 0; h < kGroupHeads; ++h) {
    m_run[h] = -INFINITY;
    l_run[h] = 0.f;
#pragma unroll
    for (int d = 0; d < 8; ++d) o[h][d] = 0.f;
  }

  for (bool first = true; t0 < c_end; t0 += kWarps * kTile, first = false) {
    if (!first) {
      const uint4* kp = reinterpret_cast<const uint4*>(kbase + (size_t)min(t0 + lane, last_tok) * kHeadDim);
#pragma unroll
      for (int i = 0; i < 8; ++i) kr[i] = ldg_nc_u128(kp + i);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        vr[i] = ldg_nc_u128(vbase + (size_t)min(t0 + 4 * i + vt, last_tok) * kHeadDim + vd);
    }
    if (t0 + kTile <= c_begin) continue;  // tile entirely left of the row's first token
    const int t = t0 + lane;
    const bool valid = t >= c_begin && t < c_end;

    float s[kGroupHeads];
#pragma unroll
    for (int h = 0; h < kGroupHeads; ++h) s[h] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const half2* h2 = reinterpret_cast<const half2*>(&kr[i]);
      float kf[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h2[j]);
        kf[2 * j] = f.x;
        kf[2 * j + 1] = f.y;
      }
#pragma unroll
      for (int h = 0; h < kGroupHeads; ++h) {
        const float4 qa = *reinterpret_cast<const float4*>(&q_s[h * kHeadDim + 8 * i]);
        const float4 qb = *reinterpret_cast<const float4*>(&q_s[h * kHeadDim + 8 * i + 4]);
        s[h] = fmaf(kf[0], qa.x, s[h]);
        s[h] = fmaf(kf[1], qa.y, s[h]);
        s[h] = fmaf(kf[2], qa.z, s[h]);
        s[h] = fmaf(kf[3], qa.w, s[h]);
        s[h] = fmaf(kf[4], qb.x, s[h]);
        s[h] = fmaf(kf[5], qb.y, s[h]);
        s[h] = fmaf(kf[6], qb.z, s[h]);
        s[h] = fmaf(kf[7], qb.w, s[h]);
      }
    }
    float alpha[kGroupHeads];
#pragma unroll
    for (int h = 0; h < kGroupHeads; ++h) {
      const float sv = valid ? s[h] : -INFINITY;
      const float m_new = fmaxf(m_run[h], warp_max(sv));  // finite: the tile has >= 1 token
      alpha[h] = (m_run[h] == -INFINITY) ? 0.f : __expf(m_run[h] - m_new);
      const float p = valid ? __expf(sv - m_new) : 0.f;
      l_run[h] = l_run[h] * alpha[h] + p;  // per-lane partial, summed at the end
      m_run[h] = m_new;
      p_s[warp][h][lane] = p;
    }
    __syncwarp();
#pragma unroll
    for (int h = 0; h < kGroupHeads; ++h)
#pragma unroll
      for (int d = 0; d < 8; ++d) o[h][d] *= alpha[h];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int tt = 4 * i + vt;
      const half2* h2 = reinterpret_cast<const half2*>(&vr[i]);
      float vf[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h2[j]);
        vf[2 * j] = f.x;
        vf[2 * j + 1] = f.y;
      }
#pragma unroll
      for (int h = 0; h < kGroupHeads; ++h) {
        const float p = p_s[warp][h][tt];  // 0 for tokens outside the range
#pragma unroll
        for (int d = 0; d < 8; ++d) o[h][d] = fmaf(p, vf[d], o[h][d]);
      }
    }
    __syncwarp();
  }

  // Warp totals: l over lanes; o over the four token classes (lane bits 3,4).
#pragma unroll
  for (int h = 0; h < kGroupHeads; ++h) {
    l_run[h] = warp_sum(l_run[h]);
#pragma unroll
    for (int d = 0; d < 8; ++d) {
      float v = o[h][d];
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      o[h][d] = v;
    }
    if (lane < 8) {
#pragma unroll
      for (int d = 0; d < 8; ++d) o_s[warp][h][lane * 8 + d] = o[h][d];
    }
    if (lane == 0) {
      m_s[warp][h] = m_run[h];
      l_s[warp][h] = l_run[h];
    }
  }
  __syncthreads();

  // Merge the 8 warps; thread -> (head, dim).
  for (int idx = tid; idx < kGroupHeads * kHeadDim; idx += kWarps * 32) {
    const int h = idx >> 6, d = idx & 63;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) m = fmaxf(m, m_s[w][h]);
    float num = 0.f, den = 0.f;
    if (m != -INFINITY) {
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float e = (m_s[w][h] == -INFINITY) ? 0.f : __expf(m_s[w][h] - m);
        den += e * l_s[w][h];
        num += e * o_s[w][h][d];
      }
    }
    const int qh = kvh * kGroupHeads + h;
    if (a.splits == 1) {
      a.out[((size_t)b * kHeads + qh) * kHeadDim + d] =
          __float2half_rn(m == -INFINITY ? 0.f : num / den);
    } else {
      const size_t row = ((size_t)b * kHeads + qh) * a.splits + split;
      a.o_part[row * kHeadDim + d] = num;
      if (d == 0) {
        a.m_part[row] = m;
        a.l_part[row] = den;
      }
    }
  }
  if (a.splits == 1 || a.consumer_merge) return;

  merge_splits_last_cta(a, b, kvh, split, &last_flag);
}



// ---------------------------------------------------------------------------
// Latency variant for short contexts at small batch (one decode step of a few
// rows): ONE WARP owns 64 tokens of one (row, kv head); the arithmetic is in
// attn_warp.cuh.
//
// Inside the decode chain (a.prefetch) the cache tile is requested BEFORE the
// dependency wait, so it is in registers when the query arrives.  That is sound
// for every row except the one the preceding qkv kernel appends in this very
// step, which the lanes that hold it fetch again after the wait.  Rows appended
// by earlier steps are complete as soon as the step counter (advanced by the
// last CTA of the lm_head kernel) shows the current step; the counter is read
// with acquire semantics before the tile is requested and again after the wait,
// and if the two differ the whole tile is fetched again.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(32) attn_decode_warp_kernel(const AttnArgs a) {
  __shared__ int last_flag;
  const int lane = threadIdx.x;
  const int g = lane >> 2, c = lane & 3;  // fragment row (head) and column pair
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  int slot = b;
  if (a.pos != nullptr) slot = a.rows[b];  // the row -> slot map is not written inside the chain
  const half* kbase = a.k + (size_t)slot * a.stride_b + (size_t)kvh * a.stride_h;
  const half* vbase = a.v + (size_t)slot * a.stride_b + (size_t)kvh * a.stride_h;
  const int last_tok = a.s_cap - 1;
  const int t0 = split * kWarpChunk;
  pdl_trigger_early();

  WarpTile tile;
  int epoch0 = 0;
  const bool prefetch = a.prefetch != 0 && a.epoch != nullptr;
  if (prefetch) {
    epoch0 = ld_acquire_s32(a.epoch);
    warp_tile_request(tile, kbase, vbase, t0, last_tok, g, c);
  }
  pdl_wait();

  int t_begin = 0, t_end = a.s_cap;
  int fresh = -1;  // row appended by the preceding kernel of the chain
  bool refetch = !prefetch;
  if (a.pos != nullptr) {
    t_end = __ldcg(a.pos + slot) + 1;
    fresh = t_end - 1;
    if (prefetch) refetch = __ldcg(a.epoch) != epoch0;
  } else {
    if (a.start != nullptr) t_begin = a.start[b];
    if (a.end != nullptr) t_end = a.end[b];
  }
  uint32_t qa0[4], qa2[4];
  warp_q_fragments(qa0, qa2, a.q + ((size_t)b * kHeads + kvh * kGroupHeads) * kHeadDim, g, c);
  warp_tile_refetch(tile, kbase, vbase, t0, last_tok, g, c, refetch, fresh);
  if (t_end > a.s_cap) t_end = a.s_cap;
  if (t_begin < 0) t_begin = 0;
  const int c_begin = max(t_begin, t0);
  const int c_end = min(t_end, t0 + kWarpChunk);

  float m, l, o[8][4];
  warp_tile_attend(tile, qa0, qa2, t0, c_begin, c_end, a.scale, c, m, l, o);

  // ---- C columns 2c, 2c+1 of mma j are dims 16c + j and 16c + 8 + j of head g
  if (g < kGroupHeads) {
    const int qh = kvh * kGroupHeads + g;
    if (a.splits == 1) {
      const float inv = (m == -INFINITY || l == 0.f) ? 0.f : 1.f / l;
      half* op = a.out + ((size_t)b * kHeads + qh) * kHeadDim + 16 * c;
      uint4 lo, hi;
      lo.x = pack_half2(o[0][0] * inv, o[1][0] * inv);
      lo.y = pack_half2(o[2][0] * inv, o[3][0] * inv);
      lo.z = pack_half2(o[4][0] * inv, o[5][0] * inv);
      lo.w = pack_half2(o[6][0] * inv, o[7][0] * inv);
      hi.x = pack_half2(o[0][1] * inv, o[1][1] * inv);
      hi.y = pack_half2(o[2][1] * inv, o[3][1] * inv);
      hi.z = pack_half2(o[4][1] * inv, o[5][1] * inv);
      hi.w = pack_half2(o[6][1] * inv, o[7][1] * inv);
      *reinterpret_cast<uint4*>(op) = lo;
      *reinterpret_cast<uint4*>(op + 8) = hi;
    } else {
      const size_t row = ((size_t)b * kHeads + qh) * a.splits + split;
      float4* op = reinterpret_cast<float4*>(a.o_part + row * kHeadDim + 16 * c);
      op[0] = make_float4(o[0][0], o[1][0], o[2][0], o[3][0]);
      op[1] = make_float4(o[4][0], o[5][0], o[6][0], o[7][0]);
      op[2] = make_float4(o[0][1], o[1][1], o[2][1], o[3][1]);
      op[3] = make_float4(o[4][1], o[5][1], o[6][1], o[7][1]);
      if (c == 0) {
        a.m_part[row] = m;
        a.l_part[row] = l;
      }
    }
  }
  if (a.splits == 1 || a.consumer_merge) return;
  if (a.splits <= 32) {
    merge_splits_warp(a, b, kvh);
  } else {
    merge_splits_last_cta(a, b, kvh, split, &last_flag);
  }
}

// ---------------------------------------------------------------------------
// Throughput variant on the warp-level tensor cores.  With 7 query heads per KV
// head, q·K and p·V cost 7 FMA per byte of cache, more than the fp32 pipes can
// issue at HBM speed, so here both products are mma.m16n8k16 (fp16 in, fp32
// accumulate): heads on the M side (7 of 16 rows used), tokens / dims on N.
// No operand goes through shared memory:
//   * K: a lane loads 32 contiguous bytes of one token row (coalesced 16-byte
//     loads).  The mma's k index is mapped to head dims so that those 32 bytes
//     are exactly the lane's B fragments of the four k steps; the Q fragments
//     use the same mapping.
//   * P: the score fragment of two 8-token blocks is already the A fragment of
//     one 16-token k step (scores stay in registers).
//   * V: a lane loads 16 bytes (8 dims) of four token rows and pairs the rows
//     with byte permutes into B fragments; the n index is mapped to dims so the
//     eight mma of a k step cover all 64 dims.
// Softmax bookkeeping is fp32 per head (online rescale per 32-token tile).
// 4 warps per CTA, tiles of 32 tokens strided over the warps.
// ---------------------------------------------------------------------------
// kMmaWarps = 4 or 8 warps per CTA: 8 (256 tokens per pass) once a CTA's token range is long
// (measured: 0.93 instead of 0.85 of the copy bandwidth at 256 rows x 32768 tokens), 4 for
// shorter ranges, where more and smaller CTAs fill the machine better.
template <int kMmaWarps>
__global__ void __launch_bounds__(kMmaWarps * 32) attn_decode_mma_kernel(const AttnArgs a) {
  __shared__ float m_s[kMmaWarps][kGroupHeads];
  __shared__ float l_s[kMmaWarps][kGroupHeads];
  __shared__ __align__(16) float o_s[kMmaWarps][kGroupHeads][kHeadDim];
  __shared__ int last_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;  // fragment row (head) and column pair
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  int slot = b;
  if (a.pos != nullptr) slot = a.rows[b];
  pdl_trigger_early();
  pdl_wait();

  int t_begin = 0, t_end = a.s_cap;
  if (a.pos != nullptr) {
    t_end = __ldcg(a.pos + slot) + 1;
  } else {
    if (a.start != nullptr) t_begin = a.start[b];
    if (a.end != nullptr) t_end = a.end[b];
  }
  if (t_end > a.s_cap) t_end = a.s_cap;
  if (t_begin < 0) t_begin = 0;
  const int c_begin = max(t_begin, split * a.chunk);
  const int c_end = min(t_end, (split + 1) * a.chunk);
  const int last_tok = a.s_cap - 1;

  // Q fragments: head g (rows 7..15 of the tile are zero), dims 16c + 4ks + {0,1} | {2,3}
  uint32_t qa0[4], qa2[4];
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    qa0[ks] = qa2[ks] = 0u;
    if (g < kGroupHeads) {
      const half* qp = a.q + ((size_t)b * kHeads + kvh * kGroupHeads + g) * kHeadDim + 16 * c + 4 * ks;
      const uint2 u = *reinterpret_cast<const uint2*>(qp);
      qa0[ks] = u.x;
      qa2[ks] = u.y;
    }
  }
  const half* kbase = a.k + (size_t)slot * a.stride_b + (size_t)kvh * a.stride_h;
  const half* vbase = a.v + (size_t)slot * a.stride_b + (size_t)kvh * a.stride_h;

  float m_run = -INFINITY, l_run = 0.f;  // head g (replicated over the 4 lanes of the row)
  float o[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

  const int tile0 = (split * a.chunk) & ~31;  // tiles are aligned to 32 tokens
  for (int t0 = tile0 + warp * 32; t0 < c_end; t0 += kMmaWarps * 32) {
    if (t0 + 32 <= c_begin) continue;
    // ---- loads: K rows t0 + 8nb + g, bytes [32c, 32c+32); V rows t0 + 16j + 2c + {0,1,8,9}, dims 8g..8g+7
    uint4 kr[4][2], vr[2][4];
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
      const uint4* kp = reinterpret_cast<const uint4*>(kbase + (size_t)min(t0 + 8 * nb + g, last_tok) * kHeadDim + 16 * c);
      kr[nb][0] = ldg_nc_u128(kp);
      kr[nb][1] = ldg_nc_u128(kp + 1);
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int tb = t0 + 16 * j + 2 * c;
      vr[j][0] = ldg_nc_u128(vbase + (size_t)min(tb, last_tok) * kHeadDim + 8 * g);
      vr[j][1] = ldg_nc_u128(vbase + (size_t)min(tb + 1, last_tok) * kHeadDim + 8 * g);
      vr[j][2] = ldg_nc_u128(vbase + (size_t)min(tb + 8, last_tok) * kHeadDim + 8 * g);
      vr[j][3] = ldg_nc_u128(vbase + (size_t)min(tb + 9, last_tok) * kHeadDim + 8 * g);
    }
    // ---- scores: S[head g][token t0 + 8nb + 2c + {0,1}]
    float sc[4][2];
    float m_tile = -INFINITY;
    {
      float d[4][4];
#pragma unroll
      for (int nb = 0; nb < 4; ++nb) d[nb][0] = d[nb][1] = d[nb][2] = d[nb][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {  // k steps outermost: consecutive mma are independent
#pragma unroll
        for (int nb = 0; nb < 4; ++nb) {
          const uint32_t* u = reinterpret_cast<const uint32_t*>(&kr[nb][0]);
          mma16816(d[nb], qa0[ks], 0u, qa2[ks], 0u, u[2 * ks], u[2 * ks + 1]);
        }
      }
#pragma unroll
      for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int t = t0 + 8 * nb + 2 * c + e;
          const float v = (t >= c_begin && t < c_end) ? d[nb][e] * a.scale : -INFINITY;
          sc[nb][e] = v;
          m_tile = fmaxf(m_tile, v);
        }
      }
    }
    m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 1));
    m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 2));
    const float m_new = fmaxf(m_run, m_tile);  // the tile holds at least one token of the range
    const float alpha = (m_run == -INFINITY) ? 0.f : __expf(m_run - m_new);
    uint32_t pa[2][2];  // P as A fragments: [k step of 16 tokens][a0 | a2]
    float l_add = 0.f;
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
      const float p0 = (sc[nb][0] == -INFINITY) ? 0.f : __expf(sc[nb][0] - m_new);
      const float p1 = (sc[nb][1] == -INFINITY) ? 0.f : __expf(sc[nb][1] - m_new);
      const half2 ph = __floats2half2_rn(p0, p1);
      // the row sum uses the rounded probabilities that multiply V
      l_add += __low2float(ph) + __high2float(ph);
      pa[nb >> 1][nb & 1] = *reinterpret_cast<const uint32_t*>(&ph);
    }
    l_run = l_run * alpha + l_add;
    m_run = m_new;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o[j][0] *= alpha;
      o[j][1] *= alpha;
    }
    // ---- O[head g][dims] += P V ; mma j covers dims {8n + j}: lane n = g supplies dim 8g + j
#pragma unroll
    for (int jk = 0; jk < 2; ++jk) {
      const uint32_t* r0 = reinterpret_cast<const uint32_t*>(&vr[jk][0]);  // token 2c
      const uint32_t* r1 = reinterpret_cast<const uint32_t*>(&vr[jk][1]);  // token 2c + 1
      const uint32_t* r2 = reinterpret_cast<const uint32_t*>(&vr[jk][2]);  // token 2c + 8
      const uint32_t* r3 = reinterpret_cast<const uint32_t*>(&vr[jk][3]);  // token 2c + 9
#pragma unroll
      for (int w = 0; w < 4; ++w) {  // word w holds dims 8g + 2w, 8g + 2w + 1
        const uint32_t b0_lo = __byte_perm(r0[w], r1[w], 0x5410), b0_hi = __byte_perm(r0[w], r1[w], 0x7632);
        const uint32_t b1_lo = __byte_perm(r2[w], r3[w], 0x5410), b1_hi = __byte_perm(r2[w], r3[w], 0x7632);
        mma16816(o[2 * w], pa[jk][0], 0u, pa[jk][1], 0u, b0_lo, b1_lo);
        mma16816(o[2 * w + 1], pa[jk][0], 0u, pa[jk][1], 0u, b0_hi, b1_hi);
      }
    }
  }

  // ---- warp state -> shared memory in the layout of the scalar kernels
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  if (g < kGroupHeads) {
    if (c == 0) {
      m_s[warp][g] = m_run;
      l_s[warp][g] = l_run;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {  // C columns 2c, 2c+1 of mma j are dims 16c + j and 16c + 8 + j
      o_s[warp][g][16 * c + j] = o[j][0];
      o_s[warp][g][16 * c + 8 + j] = o[j][1];
    }
  }
  __syncthreads();

  for (int idx = tid; idx < kGroupHeads * kHeadDim; idx += kMmaWarps * 32) {
    const int h = idx >> 6, d = idx & 63;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) m = fmaxf(m, m_s[w][h]);
    float num = 0.f, den = 0.f;
    if (m != -INFINITY) {
#pragma unroll
      for (int w = 0; w < kMmaWarps; ++w) {
        const float e = (m_s[w][h] == -INFINITY) ? 0.f : __expf(m_s[w][h] - m);
        den += e * l_s[w][h];
        num += e * o_s[w][h][d];
      }
    }
    const int qh = kvh * kGroupHeads + h;
    if (a.splits == 1) {
      a.out[((size_t)b * kHeads + qh) * kHeadDim + d] = __float2half_rn(m == -INFINITY ? 0.f : num / den);
    } else {
      const size_t row = ((size_t)b * kHeads + qh) * a.splits + split;
      a.o_part[row * kHeadDim + d] = num;
      if (d == 0) {
        a.m_part[row] = m;
        a.l_part[row] = den;
      }
    }
  }
  if (a.splits == 1 || a.consumer_merge) return;
  merge_splits_last_cta(a, b, kvh, split, &last_flag);
}

}  // namespace

cudaError_t launch_attn(const AttnArgs& a, int batch, cudaStream_t s, bool pdl) {
  dim3 grid(a.splits, kKvHeads, batch);
  if (a.small) return launch(attn_decode_warp_kernel, grid, dim3(32), 0, s, pdl, a);
  if (a.use_mma) {
    if (a.chunk >= 2048) return launch(attn_decode_mma_kernel<8>, grid, dim3(256), 0, s, pdl, a);
    return launch(attn_decode_mma_kernel<4>, grid, dim3(128), 0, s, pdl, a);
  }
  return launch(attn_decode_kernel, grid, dim3(kWarps * 32), 0, s, pdl, a);
}

}  // namespace quic

using namespace quic;

extern "C" int32_t quic_attn_pick_splits(int32_t b, int32_t s_max) {
  if (b < 1) b = 1;
  // Small problems: the latency variant, one warp per 64 tokens.
  if ((int64_t)b * s_max < 8192 && s_max <= 32 * kWarpChunk) return (s_max + kWarpChunk - 1) / kWarpChunk;
  // Enough CTAs for several per SM (the kernels keep 3-4 CTAs of 4-8 warps resident), at
  // least 256 tokens per CTA, at most 64 splits.
  int by_len = (s_max + 255) / 256;
  int want = (1184 + 2 * b - 1) / (2 * b);
  int s = want < by_len ? want : by_len;
  if (s < 1) s = 1;
  if (s > 64) s = 64;
  return s;
}

extern "C" int64_t quic_attn_scratch_bytes(int32_t b, int32_t splits) {
  if (b < 1 || splits < 1) return 0;
  int64_t counters = counter_bytes(b);
  int64_t rows = (int64_t)b * kHeads * splits;
  return counters + rows * kHeadDim * 4 + 2 * ((rows * 4 + 255) / 256 * 256);
}

namespace quic {
// Carves the scratch block; shared with the decode step.
void attn_carve_scratch(void* scratch, int b, int splits, AttnArgs* a) {
  char* p = static_cast<char*>(scratch);
  int64_t counters = counter_bytes(b);
  int64_t rows = (int64_t)b * kHeads * splits;
  int64_t ml = (rows * 4 + 255) / 256 * 256;
  a->counters = reinterpret_cast<int32_t*>(p);
  a->o_part = reinterpret_cast<float*>(p + counters);
  a->m_part = reinterpret_cast<float*>(p + counters + rows * kHeadDim * 4);
  a->l_part = reinterpret_cast<float*>(p + counters + rows * kHeadDim * 4 + ml);
}
}  // namespace quic

extern "C" int quic_attn_decode(const void* q, const void* k, const void* v, int64_t stride_b,
                                int64_t stride_h, const int32_t* start, const int32_t* end,
                                int32_t s_max, float scale, void* out, int32_t b, int32_t splits,
                                void* scratch, void* stream) {
  QUIC_REQUIRE(q && k && v && out, QUIC_E_ARG, "attn_decode: null tensor");
  QUIC_REQUIRE(b >= 1 && b <= 65535 && s_max >= 1, QUIC_E_SHAPE, "attn_decode: bad batch or length");
  QUIC_REQUIRE(((uintptr_t)k % 16 == 0) && ((uintptr_t)v % 16 == 0) && stride_b % 8 == 0 &&
                   stride_h % 8 == 0,
               QUIC_E_ARG, "attn_decode: K/V must be 16-byte aligned with strides multiple of 8");
  // Left to choose (splits <= 0), 21..128 rows of up to 8192 tokens over contiguous
  // [b][2][s_max][64] planes take the streamed kernel of the decode step (one CTA per (row, KV
  // head), no scratch), where it was measured ahead of the split kernels (64 x 8192: 49 us against
  // 57; at 64 x 32768 the split kernel's 167 us stay ahead of 189).
  if (splits <= 0 && b >= 21 && b <= 128 && s_max <= 8192 && stride_h == (int64_t)s_max * kHeadDim &&
      stride_b == (int64_t)kKvHeads * s_max * kHeadDim && tc_status_words() != nullptr) {
    AttnArgs a = {};
    a.q = (const half*)q;
    a.k = (const half*)k;
    a.v = (const half*)v;
    a.stride_b = stride_b;
    a.stride_h = stride_h;
    a.start = start;
    a.end = end;
    a.s_cap = s_max;
    a.splits = 1;
    a.chunk = s_max;
    a.scale = scale > 0.f ? scale : 0.125f;
    a.out = (half*)out;
    return launch_attn_stream(a, nullptr, b, b, s_max, tc_status_words(), (cudaStream_t)stream, false);
  }
  if (splits <= 0) splits = quic_attn_pick_splits(b, s_max);
  QUIC_REQUIRE(splits <= 4096, QUIC_E_SHAPE, "attn_decode: too many splits");
  QUIC_REQUIRE(splits == 1 || scratch != nullptr, QUIC_E_ARG, "attn_decode: scratch required");
  AttnArgs a = {};
  a.q = (const half*)q;
  a.k = (const half*)k;
  a.v = (const half*)v;
  a.stride_b = stride_b;
  a.stride_h = stride_h;
  a.start = start;
  a.end = end;
  a.s_cap = s_max;
  a.splits = splits;
  a.chunk = (s_max + splits - 1) / splits;
  a.scale = scale > 0.f ? scale : 0.125f;
  a.out = (half*)out;
  a.use_mma = ((int64_t)b * s_max >= 8192) ? 1 : 0;  // enough work for the throughput variant
  a.small = (!a.use_mma && (int64_t)splits * kWarpChunk >= s_max) ? 1 : 0;
  if (splits > 1) attn_carve_scratch(scratch, b, splits, &a);
  QUIC_CUDA(launch_attn(a, b, (cudaStream_t)stream, false));
  return QUIC_OK;
}

// ---------------------------------------------------------------------------
// Allocation-free variant: the split partials and arrival counters live in a
// fixed array inside the library image instead of caller-provided scratch.
// ---------------------------------------------------------------------------
namespace {

// 8 MiB: enough for batch x splits up to 2048 (e.g. batch 64 with 32 splits,
// or batch 1 with the maximum of 64 splits).  Every GPU that loads the library
// carries this array until the process exits.
constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_attn_static_scratch[kStaticScratchBytes];

// In host code `g_attn_static_scratch` is only a handle for the runtime, not an
// address a kernel may dereference; the device address is looked up once per
// device, with that device current, and cached here.
constexpr int kMaxDevices = 64;
void* g_static_scratch_ptr[kMaxDevices] = {};

int static_scratch_for_current_device(void** out) {
  int dev = -1;
  QUIC_CUDA(cudaGetDevice(&dev));
  QUIC_REQUIRE(dev >= 0 && dev < kMaxDevices, QUIC_E_LIMIT,
               "attn_decode_noalloc: device ordinal beyond 63");
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    QUIC_CUDA(cudaGetSymbolAddress(&p, g_attn_static_scratch));
    QUIC_REQUIRE(p != nullptr, QUIC_E_CUDA, "attn_decode_noalloc: no address for the static scratch");
    g_static_scratch_ptr[dev] = p;
  }
  *out = g_static_scratch_ptr[dev];
  return QUIC_OK;
}

}  // namespace

extern "C" int64_t quic_attn_decode_noalloc_max_bytes(void) { return (int64_t)kStaticScratchBytes; }

extern "C" int quic_attn_decode_noalloc(const void* q, const void* k, const void* v,
                                        int64_t stride_b, int64_t stride_h, const int32_t* start,
                                        const int32_t* end, int32_t s_max, float scale, void* out,
                                        int32_t b, int32_t splits, void* stream) {
  QUIC_REQUIRE(b >= 1 && s_max >= 1, QUIC_E_SHAPE, "attn_decode_noalloc: bad batch or length");
  if (splits <= 0) splits = quic_attn_pick_splits(b, s_max);
  const int64_t need = quic_attn_scratch_bytes(b, splits);
  if (splits > 1 && need > (int64_t)kStaticScratchBytes)
    return fail(QUIC_E_LIMIT,
                "attn_decode_noalloc: batch x splits needs more than the 8 MiB built-in scratch "
                "(14*64*4 bytes per batch row per split); use fewer splits or quic_attn_decode");
  void* scratch = nullptr;
  if (splits > 1) {
    int rc = static_scratch_for_current_device(&scratch);
    if (rc != QUIC_OK) return rc;
    // The array keeps whatever the previous call left.  Only the arrival
    // counters must start at zero; partials are fully rewritten before use.
    QUIC_CUDA(cudaMemsetAsync(scratch, 0, (size_t)b * kKvHeads * sizeof(int32_t),
                              (cudaStream_t)stream));
  }
  return quic_attn_decode(q, k, v, stride_b, stride_h, start, end, s_max, scale, out, b, splits,
                          scratch, stream);
}

