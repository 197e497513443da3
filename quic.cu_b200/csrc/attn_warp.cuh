// One warp's share of decode attention: 64 cached tokens of one (row, KV head) against the
// 7 query heads of the group, both products on mma.sync.m16n8k16 (fp16 in, fp32 accumulate).
//
// Fragment mappings (g = lane >> 2 is the fragment row = query head, c = lane & 3):
//   * q.K: heads on the M side (rows 7..15 are zero), 8 tokens per mma on N, head dims on K.
//     The mma's k index is mapped to head dims so that the 32 contiguous bytes of a token
//     row a lane loads (two 16-byte loads) are exactly its B fragments of the four k steps:
//     lane (g, c) loads token t0 + 8nb + g, dims 16c .. 16c+15; the Q fragments use the same
//     mapping (dims 16c + 4ks + {0,1} | {2,3}).
//   * P: the score fragments of two 8-token blocks are already the A fragment of one
//     16-token k step, so probabilities never leave registers.
//   * p.V: tokens on K, dims on N.  A lane loads 16 bytes (dims 8g .. 8g+7) of the token rows
//     t0 + 16j + 2c + {0, 1, 8, 9} and pairs rows with byte permutes; mma j of a k step
//     covers dims {8n + j}, lane n = g supplying dim 8g + j, so C columns 2c, 2c+1 of mma j
//     are dims 16c + j and 16c + 8 + j of head g.
// No shared memory, no barrier, one softmax pass: row maximum and sum cost four shuffles.
#pragma once
#include "common.cuh"

namespace quic {

constexpr int kWarpChunk = 64;  // tokens per warp tile

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_cg_u128(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t pack_half2(float x, float y) {
  const half2 h = __floats2half2_rn(x, y);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ int ld_acquire_s32(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// The K and V tile of a warp in registers (128 per lane).
struct WarpTile {
  uint4 kr[8][2];  // K rows t0 + 8nb + g, bytes [32c, 32c + 32)
  uint4 vr[4][4];  // V rows t0 + 16j + 2c + {0,1,8,9}, dims 8g .. 8g+7
};

// Early request of the whole tile (non-coherent path, no L1 allocation); rows beyond the
// cache are clamped, masking happens in warp_tile_attend.
__device__ __forceinline__ void warp_tile_request(WarpTile& t, const half* kbase, const half* vbase, int t0,
                                                  int last_tok, int g, int c) {
#pragma unroll
  for (int nb = 0; nb < 8; ++nb) {
    const uint4* kp = reinterpret_cast<const uint4*>(kbase + (size_t)min(t0 + 8 * nb + g, last_tok) * kHeadDim + 16 * c);
    t.kr[nb][0] = ldg_nc_u128(kp);
    t.kr[nb][1] = ldg_nc_u128(kp + 1);
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int tb = t0 + 16 * j + 2 * c;
    t.vr[j][0] = ldg_nc_u128(vbase + (size_t)min(tb, last_tok) * kHeadDim + 8 * g);
    t.vr[j][1] = ldg_nc_u128(vbase + (size_t)min(tb + 1, last_tok) * kHeadDim + 8 * g);
    t.vr[j][2] = ldg_nc_u128(vbase + (size_t)min(tb + 8, last_tok) * kHeadDim + 8 * g);
    t.vr[j][3] = ldg_nc_u128(vbase + (size_t)min(tb + 9, last_tok) * kHeadDim + 8 * g);
  }
}

// Coherent (L2) fetch of every row (`all`) or only of the row `fresh` that the preceding
// kernel of the chain appended after the early request was made.
__device__ __forceinline__ void warp_tile_refetch(WarpTile& t, const half* kbase, const half* vbase, int t0,
                                                  int last_tok, int g, int c, bool all, int fresh) {
#pragma unroll
  for (int nb = 0; nb < 8; ++nb) {
    const int row = t0 + 8 * nb + g;
    if (all || row == fresh) {
      const uint4* kp = reinterpret_cast<const uint4*>(kbase + (size_t)min(row, last_tok) * kHeadDim + 16 * c);
      t.kr[nb][0] = ld_cg_u128(kp);
      t.kr[nb][1] = ld_cg_u128(kp + 1);
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int row = t0 + 16 * j + 2 * c + (r & 1) + 8 * (r >> 1);
      if (all || row == fresh) t.vr[j][r] = ld_cg_u128(vbase + (size_t)min(row, last_tok) * kHeadDim + 8 * g);
    }
  }
}

// Q fragments of head g of the group (zero for g >= 7): q points at the group's first head.
__device__ __forceinline__ void warp_q_fragments(uint32_t (&qa0)[4], uint32_t (&qa2)[4], const half* q, int g, int c) {
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    qa0[ks] = qa2[ks] = 0u;
    if (g < kHeads / kKvHeads) {
      const uint2 u = __ldcg(reinterpret_cast<const uint2*>(q + (size_t)g * kHeadDim + 16 * c + 4 * ks));
      qa0[ks] = u.x;
      qa2[ks] = u.y;
    }
  }
}

// Softmax-weighted sum over the tokens [c_begin, c_end) of the tile that starts at t0:
// m = row maximum of the scaled scores (-inf when no token is in range), l = sum of the
// fp16-rounded probabilities exp(s - m) (the values that multiply V), o = sum of p * V,
// un-normalised; o[j][0], o[j][1] are dims 16c + j, 16c + 8 + j of head g.
__device__ __forceinline__ void warp_tile_attend(const WarpTile& t, const uint32_t (&qa0)[4],
                                                 const uint32_t (&qa2)[4], int t0, int c_begin, int c_end,
                                                 float scale, int c, float& m_out, float& l_out,
                                                 float (&o)[8][4]) {
  // scores: S[head g][token t0 + 8nb + 2c + {0,1}]  (k steps outermost: consecutive mma
  // belong to different accumulators)
  float sc[8][2];
  float m = -INFINITY;
  {
    float d[8][4];
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) d[nb][0] = d[nb][1] = d[nb][2] = d[nb][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) {
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&t.kr[nb][0]);
        mma16816(d[nb], qa0[ks], 0u, qa2[ks], 0u, u[2 * ks], u[2 * ks + 1]);
      }
    }
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int tok = t0 + 8 * nb + 2 * c + e;
        const float v = (tok >= c_begin && tok < c_end) ? d[nb][e] * scale : -INFINITY;
        sc[nb][e] = v;
        m = fmaxf(m, v);
      }
    }
  }
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
  uint32_t pa[4][2];  // P as A fragments: [k step of 16 tokens][a0 | a2]
  float l = 0.f;
#pragma unroll
  for (int nb = 0; nb < 8; ++nb) {
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
  for (int jk = 0; jk < 4; ++jk) {
    const uint32_t* r0 = reinterpret_cast<const uint32_t*>(&t.vr[jk][0]);  // token 2c
    const uint32_t* r1 = reinterpret_cast<const uint32_t*>(&t.vr[jk][1]);  // token 2c + 1
    const uint32_t* r2 = reinterpret_cast<const uint32_t*>(&t.vr[jk][2]);  // token 2c + 8
    const uint32_t* r3 = reinterpret_cast<const uint32_t*>(&t.vr[jk][3]);  // token 2c + 9
#pragma unroll
    for (int w = 0; w < 4; ++w) {  // word w holds dims 8g + 2w, 8g + 2w + 1
      const uint32_t b0_lo = __byte_perm(r0[w], r1[w], 0x5410), b0_hi = __byte_perm(r0[w], r1[w], 0x7632);
      const uint32_t b1_lo = __byte_perm(r2[w], r3[w], 0x5410), b1_hi = __byte_perm(r2[w], r3[w], 0x7632);
      mma16816(o[2 * w], pa[jk][0], 0u, pa[jk][1], 0u, b0_lo, b1_lo);
      mma16816(o[2 * w + 1], pa[jk][0], 0u, pa[jk][1], 0u, b0_hi, b1_hi);
    }
  }
  m_out = m;
  l_out = l;
}

// The CTA that arrives last at the per-(row, kv head) counter merges the split partials of
// the group's 7 heads, writes the fp16 output and re-arms the counter.  No CTA waits.
// Partials are fetched 16 splits at a time with every load in flight before the first use.
// (Args = AttnArgs of decode_kernels.cuh: splits, counters, m_part / l_part / o_part, out.)
template <typename Args>
__device__ __forceinline__ void merge_splits_last_cta(const Args& a, int b, int kvh, int split, int* last_flag_s) {
  const int tid = threadIdx.x;
  int& last_flag = *last_flag_s;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&a.counters[b * kKvHeads + kvh], 1);
    last_flag = (old == a.splits - 1);
  }
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  for (int idx = tid; idx < (kHeads / kKvHeads) * kHeadDim; idx += (int)blockDim.x) {
    const int h = idx >> 6, d = idx & 63;
    const int qh = kvh * (kHeads / kKvHeads) + h;
    const size_t row = ((size_t)b * kHeads + qh) * a.splits;
    float m = -INFINITY, num = 0.f, den = 0.f;
    for (int s0 = 0; s0 < a.splits; s0 += 16) {
      float ms[16], ls[16], os[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const bool in = s0 + j < a.splits;
        ms[j] = in ? __ldcg(a.m_part + row + s0 + j) : -INFINITY;
        ls[j] = in ? __ldcg(a.l_part + row + s0 + j) : 0.f;
        os[j] = in ? __ldcg(a.o_part + (row + s0 + j) * kHeadDim + d) : 0.f;
      }
      float mc = m;
#pragma unroll
      for (int j = 0; j < 16; ++j) mc = fmaxf(mc, ms[j]);
      if (mc == -INFINITY) continue;
      const float rescale = (m == -INFINITY) ? 0.f : __expf(m - mc);
      num *= rescale;
      den *= rescale;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float e = (ms[j] == -INFINITY) ? 0.f : __expf(ms[j] - mc);
        den += e * ls[j];
        num += e * os[j];
      }
      m = mc;
    }
    a.out[((size_t)b * kHeads + qh) * kHeadDim + d] = __float2half_rn(m == -INFINITY ? 0.f : num / den);
  }
  if (tid == 0) a.counters[b * kKvHeads + kvh] = 0;
}

}  // namespace quic
