// The four W4A16 dequant-GEMV kernels of one decoder layer at small batch.
//
// Common shape: a CTA owns 32 adjacent output columns; warp g of the CTA owns
// quantisation group g of the K range the CTA covers, lane l owns column l.
// Every lane first pulls its 16 packed words (one group, 128 weights) plus the
// scale and zero point into registers.  Those loads touch weights only, so they
// are issued BEFORE griddepcontrol.wait and overlap the tail of the previous
// kernel.  After the wait the CTA builds the activation vector in shared
// memory (residual add + RMSNorm where the layer has one), multiplies, reduces
// the K groups across warps through shared memory and applies the epilogue.
//
// Reference for the arithmetic of each piece:
//   dequant            src/quant/checkpoint.py:23-36, kernels/cuda/marlin.cu:2290-2313
//   residual + RMSNorm src/model.py:219-224, kernels/cuda/rmsnorm.cu:39-86
//   QKV bias           kernels/cuda/marlin.cu:2686-2693
//   RoPE               kernels/cuda/rope.cu:44-61
//   KV append          src/model.py:160 (DynamicCache.update)
//   SwiGLU             kernels/cuda/swiglu.cu:31-33
#include "decode_kernels.cuh"

namespace quic {

namespace {

constexpr int kQuarter = kHidden / 4;  // 224 threads cover a 896-wide row, 4 each

struct Half4 {
  half2 a, b;
};

__device__ __forceinline__ float4 half4_to_float4(Half4 h) {
  float2 x = __half22float2(h.a), y = __half22float2(h.b);
  return make_float4(x.x, x.y, y.x, y.y);
}

// Sum of `n` per-thread values over the block (blockDim multiple of 32, <= 1024).
template <int M>
__device__ __forceinline__ void block_sum(float (&v)[M], float* red /* [M][32] */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int m = 0; m < M; ++m) {
    float s = warp_sum(v[m]);
    if (lane == 0) red[m * 32 + warp] = s;
  }
  __syncthreads();
#pragma unroll
  for (int m = 0; m < M; ++m) {
    float s = lane < nwarp ? red[m * 32 + lane] : 0.0f;
    v[m] = warp_sum(s);
  }
  __syncthreads();
}

// Builds xs[m][perm_k(k)] = fp16-rounded RMSNorm(x_m)[k] as float for the M rows
// starting at row0.  x_m = src_m (+ fp16(sum of split partials)), the sum being
// rounded to fp16 before and after the add as the reference does (its linear
// outputs and its residual stream are fp16 tensors).  When xres_out is set the
// un-normalised x is written back by this CTA.
template <int M>
__device__ __forceinline__ void residual_norm_to_smem(
    float* xs, float* red, const half* const (&src)[M], const float* partial, int n_partial,
    int batch, int row0, const half* ln, float eps, half* xres_out) {
  const int t = threadIdx.x;
  float4 x[M];
  float ssq[M];
#pragma unroll
  for (int m = 0; m < M; ++m) {
    ssq[m] = 0.0f;
    x[m] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (t < kQuarter && src[m] != nullptr) {
      Half4 h = *reinterpret_cast<const Half4*>(src[m] + 4 * t);
      float4 v = half4_to_float4(h);
      if (partial != nullptr) {
        float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < n_partial; ++j) {
          const float4 q = __ldcg(reinterpret_cast<const float4*>(
              partial + ((size_t)j * batch + (row0 + m)) * kHidden + 4 * t));
          p.x += q.x; p.y += q.y; p.z += q.z; p.w += q.w;
        }
        v.x = __half2float(__float2half_rn(v.x + __half2float(__float2half_rn(p.x))));
        v.y = __half2float(__float2half_rn(v.y + __half2float(__float2half_rn(p.y))));
        v.z = __half2float(__float2half_rn(v.z + __half2float(__float2half_rn(p.z))));
        v.w = __half2float(__float2half_rn(v.w + __half2float(__float2half_rn(p.w))));
      }
      if (xres_out != nullptr) {
        Half4 o;
        o.a = __floats2half2_rn(v.x, v.y);
        o.b = __floats2half2_rn(v.z, v.w);
        *reinterpret_cast<Half4*>(xres_out + (size_t)(row0 + m) * kHidden + 4 * t) = o;
      }
      x[m] = v;
      ssq[m] = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  }
  block_sum<M>(ssq, red);
  if (t < kQuarter) {
    const float4 w = half4_to_float4(*reinterpret_cast<const Half4*>(ln + 4 * t));
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const float r = rsqrtf(ssq[m] * (1.0f / kHidden) + eps);
      float* dst = xs + m * kHidden;
      const int k = 4 * t;
      dst[perm_k(k + 0)] = __half2float(__float2half_rn(x[m].x * r * w.x));
      dst[perm_k(k + 1)] = __half2float(__float2half_rn(x[m].y * r * w.y));
      dst[perm_k(k + 2)] = __half2float(__float2half_rn(x[m].z * r * w.z));
      dst[perm_k(k + 3)] = __half2float(__float2half_rn(x[m].w * r * w.w));
    }
  }
  __syncthreads();
}

// Registers of one lane for one quantisation group of one column.
struct GroupRegs {
  uint32_t q[kWordsPerGroup];
  half2 s2;
  half2 zp;
};

__device__ __forceinline__ void load_group(GroupRegs& r, const quic_w4_t& w, int g, int n) {
  const int32_t* p = w.qw + (size_t)g * kWordsPerGroup * w.n + n;
#pragma unroll
  for (int j = 0; j < kWordsPerGroup; ++j) r.q[j] = ldg_nc_u32(p + (size_t)j * w.n);
  const half s = reinterpret_cast<const half*>(w.sc)[(size_t)g * w.n + n];
  r.s2 = __half2half2(s);
  const uint8_t zb = w.zp[(size_t)g * (w.n >> 1) + (n >> 1)];
  r.zp = zp_to_half2((zb >> (4 * (n & 1))) & 15);
}

// acc[m] += sum over the group of dequant(w) * xs_m ; xs points at the group's
// first k (perm8 order inside each slab of 8), rows `stride` floats apart.
template <int M>
__device__ __forceinline__ void group_fma(const GroupRegs& r, const float* xs, int stride,
                                          float (&acc)[M]) {
#pragma unroll
  for (int j = 0; j < kWordsPerGroup; ++j) {
    half2 w4[4];
    dequant8(r.q[j], r.zp, r.s2, w4);
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = dot8(w4, xs + m * stride + 8 * j, acc[m]);
  }
}

// ---------------------------------------------------------------------------
// K1: (residual +) RMSNorm -> QKV GEMV -> bias -> RoPE -> q buffer / KV append.
// grid (36, ceil(batch/M)), block 224.
// ---------------------------------------------------------------------------
template <int M>
__global__ void __launch_bounds__(224) qkv_kernel(const QkvArgs a) {
  __shared__ __align__(16) float xs[M * kHidden];
  __shared__ float red[7 * M * 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 32 + lane;
  const int row0 = blockIdx.y * M;

  GroupRegs gr;
  load_group(gr, a.w, warp, n);
  const half bias = a.w.bias ? reinterpret_cast<const half*>(a.w.bias)[n] : __float2half(0.f);
  pdl_launch_dependents();
  pdl_wait();

  const half* src[M];
  int slot[M], pos[M];
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const int b = row0 + m;
    src[m] = nullptr;
    slot[m] = -1;
    pos[m] = 0;
    if (b < a.rs.batch) {
      slot[m] = a.rs.rows[b];
      pos[m] = a.rs.pos[slot[m]];
      if (a.first_layer) {
        int tk = a.rs.tok[slot[m]];
        tk = tk < 0 ? 0 : (tk >= a.vocab ? a.vocab - 1 : tk);
        src[m] = a.embed + (size_t)tk * kHidden;
      } else {
        src[m] = a.xres_in + (size_t)b * kHidden;
      }
    }
  }
  residual_norm_to_smem<M>(xs, red, src, a.first_layer ? nullptr : a.partial, kDownSplits,
                           a.rs.batch, row0, a.ln, a.eps,
                           blockIdx.x == 0 ? a.xres_out : nullptr);

  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  group_fma<M>(gr, xs + warp * kGroup, kHidden, acc);
#pragma unroll
  for (int m = 0; m < M; ++m) red[(warp * M + m) * 32 + lane] = acc[m];
  __syncthreads();

  // Epilogue: warp `m` finishes batch row m.
  for (int m = warp; m < M; m += 7) {
    float v = 0.f;
#pragma unroll
    for (int g = 0; g < 7; ++g) v += red[(g * M + m) * 32 + lane];
    const int b = row0 + m;
    // fp16 linear output with bias, as the reference's GEMM writes it.
    v = __half2float(__float2half_rn(v + __half2float(bias)));
    const int head = n >> 6;        // 0..13 q, 14..15 k, 16..17 v
    const int i = n & 63;           // stored order: (pair, half)
    const int pair = i >> 1, hi = i & 1;
    const float other = __shfl_xor_sync(0xffffffffu, v, 1);
    // slot is warp-uniform per m: recompute from the arrays to stay in registers.
    int sl = -1, p = 0;
#pragma unroll
    for (int mm = 0; mm < M; ++mm)
      if (mm == m) { sl = slot[mm]; p = pos[mm]; }
    if (b >= a.rs.batch || sl < 0) continue;
    float out = v;
    if (head < kHeads + kKvHeads) {
      const int pp = p < a.max_pos ? p : a.max_pos - 1;
      const float c = __half2float(a.cos_t[(size_t)pp * 32 + pair]);
      const float s = __half2float(a.sin_t[(size_t)pp * 32 + pair]);
      const float lo = hi ? other : v, up = hi ? v : other;
      out = hi ? (lo * s + up * c) : (lo * c - up * s);
    }
    const int dim = pair + 32 * hi;
    const half o16 = __float2half_rn(out);
    if (head < kHeads) {
      a.qbuf[((size_t)b * kHeads + head) * kHeadDim + dim] = o16;
    } else if (p < a.s_max) {
      const int kvh = (head - kHeads) & 1;
      half* base = (head < kHeads + kKvHeads) ? a.kcache : a.vcache;
      base[(((size_t)sl * kKvHeads + kvh) * a.s_max + p) * kHeadDim + dim] = o16;
    }
  }
}

// ---------------------------------------------------------------------------
// K3: o_proj GEMV + residual add.  grid (28, ceil(batch/M)), block 224.
// ---------------------------------------------------------------------------
template <int M>
__global__ void __launch_bounds__(224) oproj_kernel(const OProjArgs a) {
  __shared__ __align__(16) float xs[M * kHidden];
  __shared__ float red[7 * M * 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 32 + lane;
  const int row0 = blockIdx.y * M;

  GroupRegs gr;
  load_group(gr, a.w, warp, n);
  pdl_launch_dependents();
  pdl_wait();

  {
    const int t = threadIdx.x;  // 224 threads x 4 elements
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row0 + m < a.batch)
        v = half4_to_float4(
            *reinterpret_cast<const Half4*>(a.attn + (size_t)(row0 + m) * kHidden + 4 * t));
      float* dst = xs + m * kHidden;
      dst[perm_k(4 * t + 0)] = v.x;
      dst[perm_k(4 * t + 1)] = v.y;
      dst[perm_k(4 * t + 2)] = v.z;
      dst[perm_k(4 * t + 3)] = v.w;
    }
  }
  __syncthreads();

  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  group_fma<M>(gr, xs + warp * kGroup, kHidden, acc);
#pragma unroll
  for (int m = 0; m < M; ++m) red[(warp * M + m) * 32 + lane] = acc[m];
  __syncthreads();

  for (int m = warp; m < M; m += 7) {
    const int b = row0 + m;
    if (b >= a.batch) continue;
    float v = 0.f;
#pragma unroll
    for (int g = 0; g < 7; ++g) v += red[(g * M + m) * 32 + lane];
    const float o = __half2float(__float2half_rn(v));
    const float r = __half2float(a.xres_in[(size_t)b * kHidden + n]);
    a.xres_out[(size_t)b * kHidden + n] = __float2half_rn(r + o);
  }
}

// ---------------------------------------------------------------------------
// K4: RMSNorm -> gate & up GEMV -> SwiGLU.  grid (152, ceil(batch/M)), block 224.
// Lane l owns gate column n and up column n + 4864.
// ---------------------------------------------------------------------------
template <int M>
__global__ void __launch_bounds__(224) gateup_kernel(const GateUpArgs a) {
  __shared__ __align__(16) float xs[M * kHidden];
  __shared__ float red[7 * M * 2 * 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 32 + lane;
  const int row0 = blockIdx.y * M;

  GroupRegs gg, gu;
  load_group(gg, a.w, warp, n);
  load_group(gu, a.w, warp, n + kInter);
  pdl_launch_dependents();
  pdl_wait();

  const half* src[M];
#pragma unroll
  for (int m = 0; m < M; ++m)
    src[m] = (row0 + m < a.batch) ? a.xres + (size_t)(row0 + m) * kHidden : nullptr;
  residual_norm_to_smem<M>(xs, red, src, nullptr, 0, a.batch, row0, a.ln, a.eps, nullptr);

  float ag[M], au[M];
#pragma unroll
  for (int m = 0; m < M; ++m) ag[m] = au[m] = 0.f;
  group_fma<M>(gg, xs + warp * kGroup, kHidden, ag);
  group_fma<M>(gu, xs + warp * kGroup, kHidden, au);
#pragma unroll
  for (int m = 0; m < M; ++m) {
    red[((warp * M + m) * 2 + 0) * 32 + lane] = ag[m];
    red[((warp * M + m) * 2 + 1) * 32 + lane] = au[m];
  }
  __syncthreads();

  for (int m = warp; m < M; m += 7) {
    const int b = row0 + m;
    if (b >= a.batch) continue;
    float g = 0.f, u = 0.f;
#pragma unroll
    for (int w = 0; w < 7; ++w) {
      g += red[((w * M + m) * 2 + 0) * 32 + lane];
      u += red[((w * M + m) * 2 + 1) * 32 + lane];
    }
    g = __half2float(__float2half_rn(g));
    u = __half2float(__float2half_rn(u));
    a.act[(size_t)b * kInter + n] = __float2half_rn(silu_mul(g, u));
  }
}

// ---------------------------------------------------------------------------
// K5: down GEMV, K split over kDownSplits CTAs; fp32 partials are summed by the
// consumer (the next layer's K1 or the lm_head).  grid (28, 5, ceil(batch/M)),
// block 256 (8 warps = up to 8 groups).
// ---------------------------------------------------------------------------
template <int M>
__global__ void __launch_bounds__(256) down_kernel(const DownArgs a) {
  __shared__ __align__(16) float xs[M * 8 * kGroup];
  __shared__ float red[8 * M * 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 32 + lane;
  const int ks = blockIdx.y;
  const int row0 = blockIdx.z * M;
  const int g0 = down_group_begin(ks), g1 = down_group_begin(ks + 1);
  const bool has = g0 + warp < g1;

  GroupRegs gr;
  if (has) load_group(gr, a.w, g0 + warp, n);
  pdl_launch_dependents();
  pdl_wait();

  const int kspan = (g1 - g0) * kGroup;
  for (int idx = threadIdx.x; idx < M * (kspan / 4); idx += 256) {
    const int m = idx / (kspan / 4), c = idx % (kspan / 4);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row0 + m < a.batch)
      v = half4_to_float4(*reinterpret_cast<const Half4*>(
          a.act + (size_t)(row0 + m) * kInter + g0 * kGroup + 4 * c));
    float* dst = xs + m * (8 * kGroup);
    dst[perm_k(4 * c + 0)] = v.x;
    dst[perm_k(4 * c + 1)] = v.y;
    dst[perm_k(4 * c + 2)] = v.z;
    dst[perm_k(4 * c + 3)] = v.w;
  }
  __syncthreads();

  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  if (has) group_fma<M>(gr, xs + warp * kGroup, 8 * kGroup, acc);
#pragma unroll
  for (int m = 0; m < M; ++m) red[(warp * M + m) * 32 + lane] = acc[m];
  __syncthreads();

  for (int m = warp; m < M; m += 8) {
    const int b = row0 + m;
    if (b >= a.batch) continue;
    float v = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) v += red[(g * M + m) * 32 + lane];
    a.partial[((size_t)ks * a.batch + b) * kHidden + n] = v;
  }
}

template <int M>
cudaError_t launch_qkv_m(const QkvArgs& a, cudaStream_t s, bool pdl) {
  dim3 grid(kQkvN / 32, (a.rs.batch + M - 1) / M);
  return launch(qkv_kernel<M>, grid, dim3(224), 0, s, pdl, a);
}
template <int M>
cudaError_t launch_oproj_m(const OProjArgs& a, cudaStream_t s, bool pdl) {
  dim3 grid(kHidden / 32, (a.batch + M - 1) / M);
  return launch(oproj_kernel<M>, grid, dim3(224), 0, s, pdl, a);
}
template <int M>
cudaError_t launch_gateup_m(const GateUpArgs& a, cudaStream_t s, bool pdl) {
  dim3 grid(kInter / 32, (a.batch + M - 1) / M);
  return launch(gateup_kernel<M>, grid, dim3(224), 0, s, pdl, a);
}
template <int M>
cudaError_t launch_down_m(const DownArgs& a, cudaStream_t s, bool pdl) {
  dim3 grid(kHidden / 32, kDownSplits, (a.batch + M - 1) / M);
  return launch(down_kernel<M>, grid, dim3(256), 0, s, pdl, a);
}

inline int pick_m(int batch) { return batch <= 1 ? 1 : batch <= 2 ? 2 : batch <= 4 ? 4 : 8; }

}  // namespace

#define QUIC_DISPATCH_M(fn, batch, ...)          \
  switch (pick_m(batch)) {                       \
    case 1: return fn<1>(__VA_ARGS__);           \
    case 2: return fn<2>(__VA_ARGS__);           \
    case 4: return fn<4>(__VA_ARGS__);           \
    default: return fn<8>(__VA_ARGS__);          \
  }

cudaError_t launch_qkv(const QkvArgs& a, cudaStream_t s, bool pdl) {
  QUIC_DISPATCH_M(launch_qkv_m, a.rs.batch, a, s, pdl)
}
cudaError_t launch_oproj(const OProjArgs& a, cudaStream_t s, bool pdl) {
  QUIC_DISPATCH_M(launch_oproj_m, a.batch, a, s, pdl)
}
cudaError_t launch_gateup(const GateUpArgs& a, cudaStream_t s, bool pdl) {
  QUIC_DISPATCH_M(launch_gateup_m, a.batch, a, s, pdl)
}
cudaError_t launch_down(const DownArgs& a, cudaStream_t s, bool pdl) {
  QUIC_DISPATCH_M(launch_down_m, a.batch, a, s, pdl)
}

}  // namespace quic
