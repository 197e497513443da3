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
    half* xs, float* red, const half* const (&src)[M], const float* partial, int n_partial,
    int batch, int row0, const float4 w, float eps, half* xres_out) {
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
        float4 q[kDownSplits];
#pragma unroll
        for (int j = 0; j < kDownSplits; ++j)  // all loads in flight together
          q[j] = __ldcg(reinterpret_cast<const float4*>(
              partial + ((size_t)j * batch + (row0 + m)) * kHidden + 4 * t));
#pragma unroll
        for (int j = 0; j < kDownSplits; ++j) {
          p.x += q[j].x; p.y += q[j].y; p.z += q[j].z; p.w += q[j].w;
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
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const float r = rsqrtf(ssq[m] * (1.0f / kHidden) + eps);
      half* dst = xs + m * kHidden;
      const int k = 4 * t;
      dst[perm_k(k + 0)] = __float2half_rn(x[m].x * r * w.x);
      dst[perm_k(k + 1)] = __float2half_rn(x[m].y * r * w.y);
      dst[perm_k(k + 2)] = __float2half_rn(x[m].z * r * w.z);
      dst[perm_k(k + 3)] = __float2half_rn(x[m].w * r * w.w);
    }
  }
  __syncthreads();
}

// Norm weight slice of this thread (4 of 896), loadable before griddepcontrol.wait.
__device__ __forceinline__ float4 load_ln(const half* ln) {
  if (threadIdx.x < kQuarter) return half4_to_float4(*reinterpret_cast<const Half4*>(ln + 4 * threadIdx.x));
  return make_float4(1.f, 1.f, 1.f, 1.f);
}

// Packed registers of one lane for one quantisation group of one column.  Loading
// does no arithmetic on the loaded values, so issuing it never stalls.
struct GroupRegs {
  uint32_t q[kWordsPerGroup];
  half s;
  uint8_t zb;
};

__device__ __forceinline__ void load_group(GroupRegs& r, const quic_w4_t& w, int g, int n) {
  const int32_t* p = w.qw + (size_t)g * kWordsPerGroup * w.n + n;
#pragma unroll
  for (int j = 0; j < kWordsPerGroup; ++j) r.q[j] = ldg_nc_u32(p + (size_t)j * w.n);
  r.s = reinterpret_cast<const half*>(w.sc)[(size_t)g * w.n + n];
  r.zb = w.zp[(size_t)g * (w.n >> 1) + (n >> 1)];
}

// The group's 128 weights as fp16 (q - zp) * s, 64 half2 registers.
struct GroupF16 {
  half2 w[kWordsPerGroup][4];
};

__device__ __forceinline__ void dequant_group(const GroupRegs& r, int n, GroupF16& d) {
  const half2 s2 = __half2half2(r.s);
  const half2 zp = zp_to_half2((r.zb >> (4 * (n & 1))) & 15);
#pragma unroll
  for (int j = 0; j < kWordsPerGroup; ++j) dequant8(r.q[j], zp, s2, d.w[j]);
}

// acc[m] += sum over the group of w * xs_m ; xs points at the group's first k
// (perm8 order inside each slab of 8), rows `stride` halves apart.
template <int M>
__device__ __forceinline__ void group_fma(const GroupF16& d, const half* xs, int stride, float (&acc)[M]) {
  float a4[M][4];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int p = 0; p < 4; ++p) a4[m][p] = 0.f;
#pragma unroll
  for (int j = 0; j < kWordsPerGroup; ++j)
#pragma unroll
    for (int m = 0; m < M; ++m) dot8_h(d.w[j], xs + m * stride + 8 * j, a4[m]);
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] += (a4[m][0] + a4[m][1]) + (a4[m][2] + a4[m][3]);
}

// Same, dequantising on the fly from the packed registers (keeps 16 instead of
// 64 weight registers; used where two groups per lane are live).
template <int M>
__device__ __forceinline__ void group_fma_packed(const GroupRegs& r, int n, const half* xs, int stride,
                                                 float (&acc)[M]) {
  const half2 s2 = __half2half2(r.s);
  const half2 zp = zp_to_half2((r.zb >> (4 * (n & 1))) & 15);
  float a4[M][4];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int p = 0; p < 4; ++p) a4[m][p] = 0.f;
#pragma unroll
  for (int j = 0; j < kWordsPerGroup; ++j) {
    half2 w4[4];
    dequant8(r.q[j], zp, s2, w4);
#pragma unroll
    for (int m = 0; m < M; ++m) dot8_h(w4, xs + m * stride + 8 * j, a4[m]);
  }
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] += (a4[m][0] + a4[m][1]) + (a4[m][2] + a4[m][3]);
}

// ---------------------------------------------------------------------------
// K1: (residual +) RMSNorm -> QKV GEMV -> bias -> RoPE -> q buffer / KV append.
// grid (36, ceil(batch/M)), block 224.
// After the wait there is ONE round of dependent global loads on the critical
// path: position + residual stream + down partials are requested together; the
// cos/sin row is requested as soon as the position arrives and lands while the
// norm and the dot products run.  (Layer 0 adds the token -> embedding row hop.)
// ---------------------------------------------------------------------------
template <int M>
__global__ void __launch_bounds__(224) qkv_kernel(const QkvArgs a) {
  __shared__ __align__(16) half xs[M * kHidden];
  __shared__ float red[7 * M * 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 32 + lane;
  const int row0 = blockIdx.y * M;

  // ---- before the wait: weights, norm weights, bias, row -> slot map (none of
  // them is written by a kernel of the decode chain)
  GroupRegs gr;
  load_group(gr, a.w, warp, n);
  const float4 lnw = load_ln(a.ln);
  const half bias = a.w.bias ? reinterpret_cast<const half*>(a.w.bias)[n] : __float2half(0.f);
  int slot[M];
#pragma unroll
  for (int m = 0; m < M; ++m) slot[m] = (row0 + m < a.rs.batch) ? a.rs.rows[row0 + m] : -1;
  GroupF16 gf;
  dequant_group(gr, n, gf);
  pdl_trigger_early();
  pdl_wait();

  const half* src[M];
  int pos[M];
#pragma unroll
  for (int m = 0; m < M; ++m) {
    src[m] = nullptr;
    pos[m] = 0;
    if (slot[m] >= 0) {
      pos[m] = __ldcg(a.rs.pos + slot[m]);
      if (a.first_layer) {
        int tk = __ldcg(a.rs.tok + slot[m]);
        tk = tk < 0 ? 0 : (tk >= a.vocab ? a.vocab - 1 : tk);
        src[m] = a.embed + (size_t)tk * kHidden;
      } else {
        src[m] = a.xres_in + (size_t)(row0 + m) * kHidden;
      }
    }
  }
  // cos/sin of this lane's RoPE pair for the rows this warp will finish
  const int head = n >> 6;  // 0..13 q, 14..15 k, 16..17 v
  const int pair = (n & 63) >> 1, hi = n & 1;
  float cs[(M + 6) / 7], sn[(M + 6) / 7];
#pragma unroll
  for (int i = 0; i < (M + 6) / 7; ++i) {
    cs[i] = 1.f;
    sn[i] = 0.f;
    const int m = warp + 7 * i;
    if (m < M && head < kHeads + kKvHeads) {
      int p = 0;
#pragma unroll
      for (int mm = 0; mm < M; ++mm)
        if (mm == m) p = pos[mm];
      p = p < a.max_pos ? p : a.max_pos - 1;
      cs[i] = __half2float(a.cos_t[(size_t)p * 32 + pair]);
      sn[i] = __half2float(a.sin_t[(size_t)p * 32 + pair]);
    }
  }
  residual_norm_to_smem<M>(xs, red, src, a.first_layer ? nullptr : a.partial, kDownSplits,
                           a.rs.batch, row0, lnw, a.eps, blockIdx.x == 0 ? a.xres_out : nullptr);

  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  group_fma<M>(gf, xs + warp * kGroup, kHidden, acc);
  pdl_trigger_late();
#pragma unroll
  for (int m = 0; m < M; ++m) red[(warp * M + m) * 32 + lane] = acc[m];
  __syncthreads();

  // Epilogue: warp w finishes batch rows w, w+7.
#pragma unroll
  for (int i = 0; i < (M + 6) / 7; ++i) {
    const int m = warp + 7 * i;
    if (m >= M) break;
    float v = 0.f;
#pragma unroll
    for (int g = 0; g < 7; ++g) v += red[(g * M + m) * 32 + lane];
    // fp16 linear output with bias, as the reference's GEMM writes it.
    v = __half2float(__float2half_rn(v + __half2float(bias)));
    const float other = __shfl_xor_sync(0xffffffffu, v, 1);
    int sl = -1, p = 0;
#pragma unroll
    for (int mm = 0; mm < M; ++mm)
      if (mm == m) { sl = slot[mm]; p = pos[mm]; }
    if (sl < 0) continue;
    const int b = row0 + m;
    float out = v;
    if (head < kHeads + kKvHeads) {
      const float lo = hi ? other : v, up = hi ? v : other;
      out = hi ? (lo * sn[i] + up * cs[i]) : (lo * cs[i] - up * sn[i]);
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
// K3: (merge of the attention splits) -> o_proj GEMV -> residual add.
// grid (28, ceil(batch/M)), block 224.  With a.splits > 0 the kernel reads the
// split partials of the attention kernel and merges them itself (every CTA
// redundantly: 896 values x splits), which saves the attention kernel an atomic
// round trip and a second pass.
// ---------------------------------------------------------------------------
template <int M>
__global__ void __launch_bounds__(224) oproj_kernel(const OProjArgs a) {
  __shared__ __align__(16) half xs[M * kHidden];
  __shared__ float red[7 * M * 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 32 + lane;
  const int row0 = blockIdx.y * M;

  GroupRegs gr;
  load_group(gr, a.w, warp, n);
  GroupF16 gf;
  dequant_group(gr, n, gf);
  pdl_trigger_early();
  pdl_wait();

  {
    const int t = threadIdx.x;  // 224 threads x 4 elements
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      const int b = row0 + m;
      if (b < a.batch) {
        if (a.splits > 0) {
          const int qh = (4 * t) >> 6, d = (4 * t) & 63;
          const size_t row = ((size_t)b * kHeads + qh) * a.splits;
          // kMaxConsumerSplits splits per pass, every load of a pass in flight together; a
          // second pass (17..32 splits) folds into the running maximum / sums
          float mx = -INFINITY, den = 0.f;
          float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int base = 0; base < a.splits; base += kMaxConsumerSplits) {
            float ms[kMaxConsumerSplits], ls[kMaxConsumerSplits];
            float4 os[kMaxConsumerSplits];
#pragma unroll
            for (int s = 0; s < kMaxConsumerSplits; ++s) {
              ms[s] = -INFINITY;
              ls[s] = 0.f;
              os[s] = make_float4(0.f, 0.f, 0.f, 0.f);
              if (base + s < a.splits) {
                ms[s] = __ldcg(a.m_part + row + base + s);
                ls[s] = __ldcg(a.l_part + row + base + s);
                os[s] = __ldcg(reinterpret_cast<const float4*>(a.o_part + (row + base + s) * kHeadDim + d));
              }
            }
            float mx_new = mx;
#pragma unroll
            for (int s = 0; s < kMaxConsumerSplits; ++s) mx_new = fmaxf(mx_new, ms[s]);
            if (mx_new == -INFINITY) continue;
            const float keep = (mx == -INFINITY) ? 0.f : __expf(mx - mx_new);
            den *= keep;
            num.x *= keep; num.y *= keep; num.z *= keep; num.w *= keep;
            mx = mx_new;
#pragma unroll
            for (int s = 0; s < kMaxConsumerSplits; ++s) {
              const float e = (ms[s] == -INFINITY) ? 0.f : __expf(ms[s] - mx);
              den += e * ls[s];
              num.x += e * os[s].x; num.y += e * os[s].y; num.z += e * os[s].z; num.w += e * os[s].w;
            }
          }
          if (mx != -INFINITY) {
            // the attention output is an fp16 tensor in the reference
            v.x = __half2float(__float2half_rn(num.x / den));
            v.y = __half2float(__float2half_rn(num.y / den));
            v.z = __half2float(__float2half_rn(num.z / den));
            v.w = __half2float(__float2half_rn(num.w / den));
          }
        } else {
          v = half4_to_float4(*reinterpret_cast<const Half4*>(a.attn + (size_t)b * kHidden + 4 * t));
        }
      }
      half* dst = xs + m * kHidden;  // values are fp16 already: exact
      dst[perm_k(4 * t + 0)] = __float2half_rn(v.x);
      dst[perm_k(4 * t + 1)] = __float2half_rn(v.y);
      dst[perm_k(4 * t + 2)] = __float2half_rn(v.z);
      dst[perm_k(4 * t + 3)] = __float2half_rn(v.w);
    }
  }
  // residual values for the epilogue rows of this warp: request them now
  float resid[(M + 6) / 7];
#pragma unroll
  for (int i = 0; i < (M + 6) / 7; ++i) {
    const int m = warp + 7 * i;
    resid[i] = (m < M && row0 + m < a.batch) ? __half2float(a.xres_in[(size_t)(row0 + m) * kHidden + n]) : 0.f;
  }
  __syncthreads();

  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  group_fma<M>(gf, xs + warp * kGroup, kHidden, acc);
  pdl_trigger_late();
#pragma unroll
  for (int m = 0; m < M; ++m) red[(warp * M + m) * 32 + lane] = acc[m];
  __syncthreads();

#pragma unroll
  for (int i = 0; i < (M + 6) / 7; ++i) {
    const int m = warp + 7 * i;
    if (m >= M) break;
    const int b = row0 + m;
    if (b >= a.batch) continue;
    float v = 0.f;
#pragma unroll
    for (int g = 0; g < 7; ++g) v += red[(g * M + m) * 32 + lane];
    const float o = __half2float(__float2half_rn(v));
    a.xres_out[(size_t)b * kHidden + n] = __float2half_rn(resid[i] + o);
  }
}

// ---------------------------------------------------------------------------
// K4: RMSNorm -> gate & up GEMV (SwiGLU is applied by the consumer).
// Work unit = (tile of 32 columns, quantisation group): 152 x 7 = 1064 units,
// dealt 8 per CTA to 133 CTAs of 8 warps, so every SM gets the same amount and
// the whole kernel is one wave (152 column tiles on 148 SMs would leave four
// SMs with double work).  The 7 units of a tile span at most two CTAs; each
// writes its fp32 partial sums to gu_part[part][gate|up][row][4864] (a CTA that
// owns the whole tile writes zeros to part 1) and the down kernel adds the two
// parts, rounds to fp16 and applies SwiGLU.  grid (133, ceil(batch/M)), block 256.
// At one row the kernel is held to 128 registers: with 156 a CTA of this kernel
// and a CTA of the down kernel (127 registers, launched early by programmatic
// dependent launch to fetch its weights) did not fit one SM's register file
// together, so most of the down kernel's weight loads started only after this
// kernel had finished.
// ---------------------------------------------------------------------------
constexpr int kGuUnitsPerCta = 8;
constexpr int kGuCtas = (kInter / 32) * 7 / kGuUnitsPerCta;  // 133

template <int M>
__global__ void __launch_bounds__(256, M == 1 ? 2 : 1) gateup_kernel(const GateUpArgs a) {
  __shared__ __align__(16) half xs[M * kHidden];
  __shared__ float red[8 * M * 2 * 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int unit = blockIdx.x * kGuUnitsPerCta + warp;
  const int tile = unit / 7, g = unit % 7;
  const int n = tile * 32 + lane;
  const int row0 = blockIdx.y * M;

  GroupRegs gg, gu;
  load_group(gg, a.w, g, n);
  load_group(gu, a.w, g, n + kInter);
  const float4 lnw = load_ln(a.ln);
  // With few batch rows the dequantised weights fit in registers: do it before the wait.
  GroupF16 fg, fu;
  if (M <= 2) {
    dequant_group(gg, n, fg);
    dequant_group(gu, n + kInter, fu);
  }
  pdl_trigger_early();
  pdl_wait();

  const half* src[M];
#pragma unroll
  for (int m = 0; m < M; ++m)
    src[m] = (row0 + m < a.batch) ? a.xres + (size_t)(row0 + m) * kHidden : nullptr;
  residual_norm_to_smem<M>(xs, red, src, nullptr, 0, a.batch, row0, lnw, a.eps, nullptr);

  float ag[M], au[M];
#pragma unroll
  for (int m = 0; m < M; ++m) ag[m] = au[m] = 0.f;
  if (M <= 2) {
    group_fma<M>(fg, xs + g * kGroup, kHidden, ag);
    group_fma<M>(fu, xs + g * kGroup, kHidden, au);
  } else {
    group_fma_packed<M>(gg, n, xs + g * kGroup, kHidden, ag);
    group_fma_packed<M>(gu, n + kInter, xs + g * kGroup, kHidden, au);
  }
  pdl_trigger_late();
#pragma unroll
  for (int m = 0; m < M; ++m) {
    red[((warp * M + m) * 2 + 0) * 32 + lane] = ag[m];
    red[((warp * M + m) * 2 + 1) * 32 + lane] = au[m];
  }
  __syncthreads();

  // Warps 0 and 1 finish the (at most two) tiles this CTA touches.
  if (warp < 2) {
    const int first_unit = blockIdx.x * kGuUnitsPerCta;
    const int t = first_unit / 7 + warp;
    const int u_lo = max(7 * t, first_unit), u_hi = min(7 * t + 7, first_unit + kGuUnitsPerCta);
    if (u_lo < u_hi) {
      const int c_a = (7 * t) / kGuUnitsPerCta, c_b = (7 * t + 6) / kGuUnitsPerCta;
      const int part = blockIdx.x - c_a;
      const int col = t * 32 + lane;
      const size_t plane = (size_t)a.batch * kInter;  // one (part, stream)
      for (int m = 0; m < M; ++m) {
        const int b = row0 + m;
        if (b >= a.batch) continue;
        float sg = 0.f, su = 0.f;
        for (int u = u_lo; u < u_hi; ++u) {
          const int w = u - first_unit;
          sg += red[((w * M + m) * 2 + 0) * 32 + lane];
          su += red[((w * M + m) * 2 + 1) * 32 + lane];
        }
        float* dst = a.gu_part + (size_t)b * kInter + col;
        dst[(2 * part + 0) * plane] = sg;
        dst[(2 * part + 1) * plane] = su;
        if (c_a == c_b) {
          dst[2 * plane] = 0.f;
          dst[3 * plane] = 0.f;
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// K5: down GEMV, K split over kDownSplits CTAs; fp32 partials are summed by the
// consumer (the next layer's K1 or the lm_head).  grid (28, 5, ceil(batch/M)),
// block 256 (8 warps = up to 8 groups).
// ---------------------------------------------------------------------------
template <int M>
__global__ void __launch_bounds__(256) down_kernel(const DownArgs a) {
  __shared__ __align__(16) half xs[M * 8 * kGroup];
  __shared__ float red[8 * M * 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 32 + lane;
  const int ks = blockIdx.y;
  const int row0 = blockIdx.z * M;
  const int g0 = down_group_begin(ks), g1 = down_group_begin(ks + 1);
  const bool has = g0 + warp < g1;

  GroupRegs gr;
  GroupF16 gf;
  if (has) {
    load_group(gr, a.w, g0 + warp, n);
    dequant_group(gr, n, gf);
  }
  pdl_trigger_early();
  pdl_wait();

  // Activation slice: add the two gate/up partial planes, round to fp16 (the
  // reference's linear outputs are fp16), SwiGLU, round again.
  const int kspan = (g1 - g0) * kGroup;
  const size_t plane = (size_t)a.batch * kInter;
  for (int idx = threadIdx.x; idx < M * (kspan / 4); idx += 256) {
    const int m = idx / (kspan / 4), c = idx % (kspan / 4);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row0 + m < a.batch) {
      const float* p = a.gu_part + (size_t)(row0 + m) * kInter + g0 * kGroup + 4 * c;
      const float4 g0v = __ldcg(reinterpret_cast<const float4*>(p));
      const float4 u0v = __ldcg(reinterpret_cast<const float4*>(p + plane));
      const float4 g1v = __ldcg(reinterpret_cast<const float4*>(p + 2 * plane));
      const float4 u1v = __ldcg(reinterpret_cast<const float4*>(p + 3 * plane));
      auto act = [](float ga, float gb, float ua, float ub) {
        const float gg = __half2float(__float2half_rn(ga + gb));
        const float uu = __half2float(__float2half_rn(ua + ub));
        return silu_mul(gg, uu);
      };
      v.x = act(g0v.x, g1v.x, u0v.x, u1v.x);
      v.y = act(g0v.y, g1v.y, u0v.y, u1v.y);
      v.z = act(g0v.z, g1v.z, u0v.z, u1v.z);
      v.w = act(g0v.w, g1v.w, u0v.w, u1v.w);
    }
    half* dst = xs + m * (8 * kGroup);
    dst[perm_k(4 * c + 0)] = __float2half_rn(v.x);
    dst[perm_k(4 * c + 1)] = __float2half_rn(v.y);
    dst[perm_k(4 * c + 2)] = __float2half_rn(v.z);
    dst[perm_k(4 * c + 3)] = __float2half_rn(v.w);
  }
  __syncthreads();

  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  if (has) group_fma<M>(gf, xs + warp * kGroup, 8 * kGroup, acc);
  pdl_trigger_late();
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
  dim3 grid(kGuCtas, (a.batch + M - 1) / M);
  return launch(gateup_kernel<M>, grid, dim3(256), 0, s, pdl, a);
}
template <int M>
cudaError_t launch_down_m(const DownArgs& a, cudaStream_t s, bool pdl) {
  dim3 grid(kHidden / 32, kDownSplits, (a.batch + M - 1) / M);
  return launch(down_kernel<M>, grid, dim3(256), 0, s, pdl, a);
}

inline int pick_m(int batch) { return batch <= 1 ? 1 : batch <= 2 ? 2 : batch <= 3 ? 3 : batch <= 4 ? 4 : 8; }

}  // namespace

#define QUIC_DISPATCH_M(fn, batch, ...)          \
  switch (pick_m(batch)) {                       \
    case 1: return fn<1>(__VA_ARGS__);           \
    case 2: return fn<2>(__VA_ARGS__);           \
    case 3: return fn<3>(__VA_ARGS__);           \
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


