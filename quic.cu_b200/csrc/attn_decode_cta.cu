// GQA decode attention without global partials: one CTA of eight warps owns 512 cached tokens
// of a (row, KV head) -- every warp the 64-token tile arithmetic of attn_warp.cuh, the eight
// warps merged through shared memory -- and, beyond 512 tokens, the CTAs of a (row, KV head)
// form a thread-block cluster (up to 8 CTAs = 4096 tokens) whose partial results meet in the
// shared memory of the cluster's first CTA (distributed shared memory, one cluster barrier).
// No scratch buffer, no counter, no fence: the merge of the split-K form costs one barrier
// instead of three round trips through L2.
//
// Same mathematics as fad_decode_kernel + fad_combine_kernel of the reference
// (kernels/cuda/flash_attn_decode.cu:12,104): fp32 softmax over the tokens [start_b, end_b)
// of each row, rows without tokens give zeros (:118-121).
//
// Inside the decode chain (a.prefetch) a warp requests its cache tile BEFORE the dependency
// wait, exactly as the one-warp kernel does (see attn_decode.cu): rows appended by earlier
// steps are complete once the step counter shows the current step, the row appended by the
// preceding qkv kernel is fetched again after the wait, and a counter that moved between the
// two reads makes the warp fetch its whole tile again.
#include "attn_warp.cuh"
#include "decode_kernels.cuh"

namespace quic {
namespace {

constexpr int kGroupHeads = kHeads / kKvHeads;  // 7
constexpr int kCtaWarps = 8;

__device__ __forceinline__ void cluster_arrive_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive_release() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of `p` (a shared-memory object of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t dsmem_addr(const void* p, uint32_t rank) {
  const uint32_t local = (uint32_t)__cvta_generic_to_shared(p);
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}
__device__ __forceinline__ void st_dsmem_f32x2(uint32_t addr, float x, float y) {
  asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(x), "f"(y) : "memory");
}
__device__ __forceinline__ void st_dsmem_f32(uint32_t addr, float x) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(x) : "memory");
}

template <bool kCluster>
__global__ void __launch_bounds__(kCtaWarps * 32, 1) attn_decode_cta_kernel(const AttnArgs a) {
  __shared__ float m_s[kCtaWarps][kGroupHeads];
  __shared__ float l_s[kCtaWarps][kGroupHeads];
  __shared__ __align__(16) float o_s[kCtaWarps][kGroupHeads][kHeadDim];
  // gathered per-CTA results of the cluster (used in its first CTA)
  __shared__ float gm_s[kCluster ? 8 : 1][kGroupHeads + 1];
  __shared__ float gl_s[kCluster ? 8 : 1][kGroupHeads + 1];
  __shared__ __align__(16) float go_s[kCluster ? 8 : 1][kGroupHeads][kHeadDim];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;  // fragment row (head) and column pair
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;  // split == rank in the cluster
  int slot = b;
  if (a.pos != nullptr) slot = a.rows[b];  // the row -> slot map is not written inside the chain
  const half* kbase = a.k + (size_t)slot * a.stride_b + (size_t)kvh * a.stride_h;
  const half* vbase = a.v + (size_t)slot * a.stride_b + (size_t)kvh * a.stride_h;
  const int last_tok = a.s_cap - 1;
  const int t0 = (split * kCtaWarps + warp) * kWarpChunk;
  pdl_trigger_early();
  // every CTA of the cluster is known to run before another CTA writes into its shared memory
  if (kCluster) cluster_arrive_relaxed();

  WarpTile tile;
  int epoch0 = 0;
  const bool prefetch = a.prefetch != 0 && a.epoch != nullptr;
  if (prefetch && t0 <= last_tok) {
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
  if (t_end > a.s_cap) t_end = a.s_cap;
  if (t_begin < 0) t_begin = 0;
  const int c_begin = max(t_begin, t0);
  const int c_end = min(t_end, t0 + kWarpChunk);

  float m = -INFINITY, l = 0.f, o[8][4];
  if (c_begin < c_end) {  // warp-uniform
    uint32_t qa0[4], qa2[4];
    warp_q_fragments(qa0, qa2, a.q + ((size_t)b * kHeads + kvh * kGroupHeads) * kHeadDim, g, c);
    warp_tile_refetch(tile, kbase, vbase, t0, last_tok, g, c, refetch, fresh);
    warp_tile_attend(tile, qa0, qa2, t0, c_begin, c_end, a.scale, c, m, l, o);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  }
  // C columns 2c, 2c+1 of mma j are dims 16c + j and 16c + 8 + j of head g
  if (g < kGroupHeads) {
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

  // the eight warps' results -> one per CTA; thread -> (head, pair of dims)
  const int h = tid >> 5, d2 = tid & 31;
  float mx = -INFINITY, den = 0.f;
  float2 num = make_float2(0.f, 0.f);
  if (h < kGroupHeads) {
#pragma unroll
    for (int w = 0; w < kCtaWarps; ++w) mx = fmaxf(mx, m_s[w][h]);
    if (mx != -INFINITY) {
#pragma unroll
      for (int w = 0; w < kCtaWarps; ++w) {
        const float e = (m_s[w][h] == -INFINITY) ? 0.f : __expf(m_s[w][h] - mx);
        const float2 v = *reinterpret_cast<const float2*>(&o_s[w][h][2 * d2]);
        den = fmaf(e, l_s[w][h], den);
        num.x = fmaf(e, v.x, num.x);
        num.y = fmaf(e, v.y, num.y);
      }
    }
  }
  half* out = a.out + ((size_t)b * kHeads + kvh * kGroupHeads + h) * kHeadDim + 2 * d2;
  if (!kCluster) {
    if (h < kGroupHeads) {
      const float inv = den > 0.f ? 1.f / den : 0.f;
      *reinterpret_cast<half2*>(out) = __floats2half2_rn(num.x * inv, num.y * inv);
    }
    return;
  }

  cluster_wait_acquire();  // pairs with the arrive at the top: the first CTA runs
  if (h < kGroupHeads) {
    st_dsmem_f32x2(dsmem_addr(&go_s[split][h][2 * d2], 0), num.x, num.y);
    if (d2 == 0) {
      st_dsmem_f32(dsmem_addr(&gm_s[split][h], 0), mx);
      st_dsmem_f32(dsmem_addr(&gl_s[split][h], 0), den);
    }
  }
  cluster_arrive_release();
  cluster_wait_acquire();
  if (split != 0 || h >= kGroupHeads) return;
  const int n = a.splits;
  float gmx = -INFINITY;
  for (int s = 0; s < n; ++s) gmx = fmaxf(gmx, gm_s[s][h]);
  float gden = 0.f;
  float2 gnum = make_float2(0.f, 0.f);
  if (gmx != -INFINITY) {
    for (int s = 0; s < n; ++s) {
      const float e = (gm_s[s][h] == -INFINITY) ? 0.f : __expf(gm_s[s][h] - gmx);
      const float2 v = *reinterpret_cast<const float2*>(&go_s[s][h][2 * d2]);
      gden = fmaf(e, gl_s[s][h], gden);
      gnum.x = fmaf(e, v.x, gnum.x);
      gnum.y = fmaf(e, v.y, gnum.y);
    }
  }
  const float inv = gden > 0.f ? 1.f / gden : 0.f;
  *reinterpret_cast<half2*>(out) = __floats2half2_rn(gnum.x * inv, gnum.y * inv);
}


}  // namespace

int attn_cta_splits(int ctx) {
  const int per = kCtaWarps * kWarpChunk;
  return ctx < 1 ? 1 : (ctx + per - 1) / per;
}

// a.splits = CTAs per (row, KV head) = cluster size, 1..kAttnCtaMaxSplits, covering a.s_cap tokens.
cudaError_t launch_attn_cta(const AttnArgs& a, int batch, cudaStream_t stream, bool pdl) {
  if (a.splits < 1 || a.splits > kAttnCtaMaxSplits || a.splits * kCtaWarps * kWarpChunk < a.s_cap)
    return cudaErrorInvalidValue;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a.splits, kKvHeads, batch);
  cfg.blockDim = dim3(kCtaWarps * 32);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (a.splits > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = a.splits;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl && pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  if (a.splits > 1) return cudaLaunchKernelEx(&cfg, attn_decode_cta_kernel<true>, a);
  return cudaLaunchKernelEx(&cfg, attn_decode_cta_kernel<false>, a);
}

}  // namespace quic

using namespace quic;

extern "C" int32_t quic_attn_decode_cta_max_tokens(void) { return kAttnCtaMaxSplits * kCtaWarps * kWarpChunk; }

extern "C" int quic_attn_decode_cta(const void* q, const void* k, const void* v, int64_t stride_b,
                                    int64_t stride_h, const int32_t* start, const int32_t* end,
                                    int32_t s_max, float scale, void* out, int32_t b, void* stream) {
  QUIC_REQUIRE(q && k && v && out, QUIC_E_ARG, "attn_decode_cta: null tensor");
  QUIC_REQUIRE(b >= 1 && b <= 65535 && s_max >= 1, QUIC_E_SHAPE, "attn_decode_cta: bad batch or length");
  QUIC_REQUIRE(s_max <= quic_attn_decode_cta_max_tokens(), QUIC_E_LIMIT,
               "attn_decode_cta: at most 4096 cached tokens (eight CTAs of 512); use quic_attn_decode");
  QUIC_REQUIRE(((uintptr_t)k % 16 == 0) && ((uintptr_t)v % 16 == 0) && ((uintptr_t)q % 8 == 0) &&
                   stride_b % 8 == 0 && stride_h % 8 == 0,
               QUIC_E_ARG, "attn_decode_cta: K/V must be 16-byte aligned with strides multiple of 8");
  AttnArgs a = {};
  a.q = (const half*)q;
  a.k = (const half*)k;
  a.v = (const half*)v;
  a.stride_b = stride_b;
  a.stride_h = stride_h;
  a.start = start;
  a.end = end;
  a.s_cap = s_max;
  a.splits = attn_cta_splits(s_max);
  a.chunk = kCtaWarps * kWarpChunk;
  a.scale = scale;
  a.out = (half*)out;
  QUIC_CUDA(launch_attn_cta(a, b, (cudaStream_t)stream, false));
  return QUIC_OK;
}
