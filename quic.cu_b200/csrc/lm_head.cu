// Tied fp16 lm_head GEMV fused with the final residual + RMSNorm and the greedy
// argmax.
//
// Replaces, for one decode step, the reference's final norm
// (src/model.py:298), cuBLAS lm_head (src/model.py:301 -> kernels/cuda/gemm.cu:36)
// and torch.argmax (src/engine.py:104; tie -> lowest index, as
// kernels/cuda/sampler.cu:38-40).  Logits are rounded to fp16 before they are
// compared because the reference's logits tensor is fp16.
//
// Mapping: a warp reads two table rows (3584 contiguous bytes) per iteration,
// 7 x 16-byte loads per lane; which of the 896 dims a lane's j-th load covers
// does not depend on the row, so for one batch row the normalised activation
// sits in registers.  A CTA owns a contiguous range of row pairs; its best
// (value, index) goes to global memory and the CTA that arrives last reduces
// the per-CTA candidates, publishes the token and advances the slot state.
#include "decode_kernels.cuh"

namespace quic {
namespace {

constexpr int kThreads = 512;
constexpr int kVecPerRow = kHidden / 8;  // 112 uint4 per row
constexpr int kVecPerLane = 7;           // 224 uint4 of a row pair / 32 lanes

struct Best {
  float v;
  int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
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
__global__ void __launch_bounds__(kThreads, 1) lm_head_kernel(const LmHeadArgs a) {
  __shared__ __align__(16) half xh[M * kHidden];
  __shared__ float red[M * 32];
  __shared__ float bv_s[M][kThreads / 32];
  __shared__ int bi_s[M][kThreads / 32];
  __shared__ int last_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // blockIdx.x (fastest) walks the batch-row chunks so that CTAs reading the
  // same table rows are co-scheduled and share them through L2.
  const int row0 = blockIdx.x * M;
  const int chunk = blockIdx.y, nchunk = gridDim.y;
  const int npairs = a.vocab >> 1;
  const int p_begin = (int)((int64_t)npairs * chunk / nchunk);
  const int p_end = (int)((int64_t)npairs * (chunk + 1) / nchunk);

  // Warm the first row pairs of this CTA while the previous kernel drains.
  for (int p = p_begin + warp; p < p_end && p < p_begin + 2 * (kThreads / 32); p += kThreads / 32) {
    const char* rowp = reinterpret_cast<const char*>(a.embed) + (size_t)p * 2 * kHidden * 2;
    prefetch_l2(rowp + lane * 112);
  }
  pdl_trigger_early();
  pdl_wait();

  // ---- activation: (x + partial sums) -> RMSNorm -> xs (natural order) ----
  {
    float4 x[M];
    float ssq[M];
#pragma unroll
    for (int m = 0; m < M; ++m) {
      x[m] = make_float4(0.f, 0.f, 0.f, 0.f);
      ssq[m] = 0.f;
      const int b = row0 + m;
      if (tid < kHidden / 4 && b < a.batch) {
        if (a.x_normed != nullptr) {
          const half2* s = reinterpret_cast<const half2*>(a.x_normed + (size_t)b * kHidden + 4 * tid);
          const float2 u = __half22float2(s[0]), w = __half22float2(s[1]);
          x[m] = make_float4(u.x, u.y, w.x, w.y);
        } else {
          const half2* s = reinterpret_cast<const half2*>(a.xres_in + (size_t)b * kHidden + 4 * tid);
          const float2 u = __half22float2(s[0]), w = __half22float2(s[1]);
          float4 v = make_float4(u.x, u.y, w.x, w.y);
          if (a.partial != nullptr) {
            float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j = 0; j < kDownSplits; ++j) {
              const float4 q = __ldcg(reinterpret_cast<const float4*>(
                  a.partial + ((size_t)j * a.batch + b) * kHidden + 4 * tid));
              p.x += q.x; p.y += q.y; p.z += q.z; p.w += q.w;
            }
            v.x = __half2float(__float2half_rn(v.x + __half2float(__float2half_rn(p.x))));
            v.y = __half2float(__float2half_rn(v.y + __half2float(__float2half_rn(p.y))));
            v.z = __half2float(__float2half_rn(v.z + __half2float(__float2half_rn(p.z))));
            v.w = __half2float(__float2half_rn(v.w + __half2float(__float2half_rn(p.w))));
          }
          x[m] = v;
          ssq[m] = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
      }
    }
    if (a.x_normed == nullptr) {
      // block-wide sum of squares
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float s = warp_sum(ssq[m]);
        if (lane == 0) red[m * 32 + warp] = s;
      }
      __syncthreads();
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float s = lane < kThreads / 32 ? red[m * 32 + lane] : 0.f;
        ssq[m] = warp_sum(s);
      }
    }
    if (tid < kHidden / 4) {
      float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
      if (a.x_normed == nullptr) {
        const half2* s = reinterpret_cast<const half2*>(a.ln + 4 * tid);
        const float2 u = __half22float2(s[0]), v = __half22float2(s[1]);
        w = make_float4(u.x, u.y, v.x, v.y);
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float4 v = x[m];
        if (a.x_normed == nullptr) {
          const float r = rsqrtf(ssq[m] * (1.0f / kHidden) + a.eps);
          v.x = __half2float(__float2half_rn(v.x * r * w.x));
          v.y = __half2float(__float2half_rn(v.y * r * w.y));
          v.z = __half2float(__float2half_rn(v.z * r * w.z));
          v.w = __half2float(__float2half_rn(v.w * r * w.w));
        }
        half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);  // exact: already fp16 values
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&h0);
        pk.y = *reinterpret_cast<uint32_t*>(&h1);
        *reinterpret_cast<uint2*>(&xh[m * kHidden + 4 * tid]) = pk;
      }
    }
    __syncthreads();
  }

  // dims of this lane's j-th 16-byte piece of a row pair
  int dim[kVecPerLane];
#pragma unroll
  for (int j = 0; j < kVecPerLane; ++j) dim[j] = ((lane + 32 * j) % kVecPerRow) * 8;
  // For one batch row the activation stays in registers (as fp16 pairs).
  uint4 xr[(M == 1) ? kVecPerLane : 1];
  if (M == 1) {
#pragma unroll
    for (int j = 0; j < kVecPerLane; ++j) xr[(M == 1) ? j : 0] = *reinterpret_cast<const uint4*>(&xh[dim[j]]);
  }

  Best best[M];
#pragma unroll
  for (int m = 0; m < M; ++m) {
    best[m].v = -INFINITY;
    best[m].i = 0x7fffffff;
  }

  // One row pair: 7 x 16-byte pieces per lane -> two logits per batch row.
  auto consume = [&](int p, const uint4 (&wv)[kVecPerLane]) {
    float acc0[M], acc1[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc0[m] = acc1[m] = 0.f;
#pragma unroll
    for (int j = 0; j < kVecPerLane; ++j) {
      const half2* w2 = reinterpret_cast<const half2*>(&wv[j]);
      // pieces 0..111 of the pair belong to the first row
      const bool first = (j < 3) || (j == 3 && lane < 16);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        uint4 xv;
        if (M == 1) xv = xr[(M == 1) ? j : 0];
        else xv = *reinterpret_cast<const uint4*>(&xh[m * kHidden + dim[j]]);
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
      const int b = row0 + m;
      if (a.logits != nullptr && lane == 0 && b < a.batch)
        *reinterpret_cast<half2*>(a.logits + (size_t)b * a.vocab + 2 * p) = __floats2half2_rn(l0, l1);
      Best c;
      c.v = l0;
      c.i = 2 * p;
      best[m] = better(best[m], c);
      c.v = l1;
      c.i = 2 * p + 1;
      best[m] = better(best[m], c);
    }
  };

  if (M <= 2) {
    // Two row pairs (7 KB per warp) are requested before either is consumed.
    for (int p = p_begin + 2 * warp; p < p_end; p += 2 * (kThreads / 32)) {
      const bool two = p + 1 < p_end;
      const uint4* src0 = reinterpret_cast<const uint4*>(a.embed + (size_t)p * 2 * kHidden);
      const uint4* src1 = reinterpret_cast<const uint4*>(a.embed + (size_t)(two ? p + 1 : p) * 2 * kHidden);
      uint4 wa[kVecPerLane], wb[kVecPerLane];
#pragma unroll
      for (int j = 0; j < kVecPerLane; ++j) wa[j] = ldg_nc_u128(src0 + lane + 32 * j);
#pragma unroll
      for (int j = 0; j < kVecPerLane; ++j) wb[j] = ldg_nc_u128(src1 + lane + 32 * j);
      consume(p, wa);
      if (two) consume(p + 1, wb);
    }
  } else {
    for (int p = p_begin + warp; p < p_end; p += kThreads / 32) {
      const uint4* src0 = reinterpret_cast<const uint4*>(a.embed + (size_t)p * 2 * kHidden);
      uint4 wa[kVecPerLane];
#pragma unroll
      for (int j = 0; j < kVecPerLane; ++j) wa[j] = ldg_nc_u128(src0 + lane + 32 * j);
      consume(p, wa);
    }
  }

  // CTA best per batch row.
#pragma unroll
  for (int m = 0; m < M; ++m) {
    if (lane == 0) {
      bv_s[m][warp] = best[m].v;
      bi_s[m][warp] = best[m].i;
    }
  }
  __syncthreads();
  if (warp < M) {
    Best c;
    c.v = lane < kThreads / 32 ? bv_s[warp][lane] : -INFINITY;
    c.i = lane < kThreads / 32 ? bi_s[warp][lane] : 0x7fffffff;
    c = warp_best(c);
    const int b = row0 + warp;
    if (lane == 0 && b < a.batch) {
      a.best_val[(size_t)b * nchunk + chunk] = c.v;
      a.best_idx[(size_t)b * nchunk + chunk] = c.i;
    }
  }

  // Last CTA (over the whole grid) reduces the candidates of every row.
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int total = gridDim.x * gridDim.y;
    const int old = atomicAdd(a.counter, 1);
    last_flag = (old == total - 1);
  }
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  int step = 0;
  if (a.step_counter != nullptr) step = *a.step_counter;
  for (int b = warp; b < a.batch; b += kThreads / 32) {
    Best c;
    c.v = -INFINITY;
    c.i = 0x7fffffff;
    for (int i = lane; i < nchunk; i += 32) {
      Best d;
      d.v = __ldcg(a.best_val + (size_t)b * nchunk + i);
      d.i = __ldcg(a.best_idx + (size_t)b * nchunk + i);
      c = better(c, d);
    }
    c = warp_best(c);
    if (lane == 0) {
      const int token = c.i == 0x7fffffff ? 0 : c.i;
      if (a.argmax_out != nullptr) a.argmax_out[b] = token;
      if (a.rows != nullptr) {
        const int slot = a.rows[b];
        a.tok[slot] = token;
        a.pos[slot] = a.pos[slot] + 1;
        if (a.out_tokens != nullptr) a.out_tokens[(size_t)(step % a.ring) * a.n_slots + slot] = token;
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    *a.counter = 0;
    __threadfence();  // the new positions and tokens are visible before the step counter moves
    if (a.step_counter != nullptr) *a.step_counter = step + 1;
  }
}

template <int M>
cudaError_t launch_lm_head_m(const LmHeadArgs& a, int grid, cudaStream_t s, bool pdl) {
  dim3 g((a.batch + M - 1) / M, grid);
  return launch(lm_head_kernel<M>, g, dim3(kThreads), 0, s, pdl, a);
}

}  // namespace

int lm_head_grid(int vocab) {
  int pairs = vocab / 2;
  int g = 148;  // one persistent CTA per SM
  if (g > pairs) g = pairs > 0 ? pairs : 1;
  return g;
}

cudaError_t launch_lm_head(const LmHeadArgs& a, int grid, cudaStream_t s, bool pdl) {
  const int b = a.batch;
  if (b <= 1) return launch_lm_head_m<1>(a, grid, s, pdl);
  if (b <= 2) return launch_lm_head_m<2>(a, grid, s, pdl);
  if (b <= 4) return launch_lm_head_m<4>(a, grid, s, pdl);
  return launch_lm_head_m<8>(a, grid, s, pdl);
}

}  // namespace quic

using namespace quic;

extern "C" int64_t quic_lm_head_scratch_bytes(int32_t b, int32_t vocab) {
  if (b < 1 || vocab < 2) return 0;
  const int64_t per = ((int64_t)b * lm_head_grid(vocab) * 4 + 255) / 256 * 256;
  return 256 + 2 * per;
}

extern "C" int quic_lm_head_argmax(const void* x, const void* norm_w, float eps, const void* embed,
                                   int32_t vocab, int32_t b, void* logits, int64_t* out,
                                   void* scratch, void* stream) {
  QUIC_REQUIRE(x && embed && scratch, QUIC_E_ARG, "lm_head_argmax: null tensor");
  QUIC_REQUIRE(b >= 1 && b <= 8 * 65535 && vocab >= 2 && vocab % 2 == 0, QUIC_E_SHAPE,
               "lm_head_argmax: batch >= 1 and an even vocabulary are required");
  QUIC_REQUIRE(((uintptr_t)x % 8 == 0) && ((uintptr_t)embed % 16 == 0), QUIC_E_ARG,
               "lm_head_argmax: x must be 8-byte and the table 16-byte aligned");
  const int grid = lm_head_grid(vocab);
  const int64_t per = ((int64_t)b * grid * 4 + 255) / 256 * 256;
  char* base = static_cast<char*>(scratch);
  LmHeadArgs a = {};
  a.embed = (const half*)embed;
  a.batch = b;
  a.vocab = vocab;
  a.eps = eps;
  a.logits = (half*)logits;
  a.counter = reinterpret_cast<int32_t*>(base);
  a.best_val = reinterpret_cast<float*>(base + 256);
  a.best_idx = reinterpret_cast<int32_t*>(base + 256 + per);
  a.argmax_out = out;
  a.ring = 1;
  if (norm_w != nullptr) {
    a.ln = (const half*)norm_w;
    a.xres_in = (const half*)x;
  } else {
    a.x_normed = (const half*)x;
  }
  QUIC_CUDA(launch_lm_head(a, grid, (cudaStream_t)stream, false));
  return QUIC_OK;
}

