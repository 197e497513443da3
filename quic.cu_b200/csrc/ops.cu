// Stand-alone operators with the reference's per-op call shapes: RMSNorm
// (+ residual), RoPE and its tables, SwiGLU, argmax, fp16 GEMV.  They serve the
// prefill path, the per-op parity tests and callers that use the reference's
// kernel getters one op at a time; the decode step fuses all of them.
#include <math.h>

#include "decode_kernels.cuh"

namespace quic {

static thread_local char g_err[256] = "";
void set_pdl(bool on);
void set_error(const char* msg) {
  int i = 0;
  for (; msg && msg[i] && i < 255; ++i) g_err[i] = msg[i];
  g_err[i] = 0;
}
static bool g_pdl = true;
bool pdl_enabled() { return g_pdl; }
void set_pdl(bool on) { g_pdl = on; }
int fail(int code, const char* msg) {
  set_error(msg);
  return code;
}

namespace {

// ---- RMSNorm (+ residual) ---------------------------------------------------
// One CTA of 224 threads per row of 896 (4 elements per thread); every global load of the
// row, the residual and the weight is requested before the first use.
// With `part` set, the row is the fp16-rounded sum of `splits` fp32 partial planes
// [splits][rows][896] (split-K output of the GEMM before it) instead of x.
__global__ void __launch_bounds__(224) rmsnorm_kernel(const half* __restrict__ x, const float* __restrict__ part,
                                                      int splits, const half* __restrict__ res,
                                                      const half* __restrict__ w, float eps,
                                                      half* __restrict__ y,
                                                      half* __restrict__ sum_out, int rows) {
  __shared__ float red[8];
  const int row = blockIdx.x, t = threadIdx.x, c = 4 * t;
  const uint2 wv = *reinterpret_cast<const uint2*>(w + c);  // weights: not produced by the chain
  pdl_launch_dependents();
  pdl_wait();
  uint2 r = make_uint2(0, 0);
  if (res != nullptr) r = *reinterpret_cast<const uint2*>(res + (size_t)row * kHidden + c);
  float2 a, b;
  if (part != nullptr) {
    float4 p[16];
#pragma unroll
    for (int s = 0; s < 16; ++s)
      p[s] = s < splits ? __ldcg(reinterpret_cast<const float4*>(part + ((size_t)s * rows + row) * kHidden + c))
                        : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < 16; ++s) {
      v.x += p[s].x; v.y += p[s].y; v.z += p[s].z; v.w += p[s].w;
    }
    a = make_float2(__half2float(__float2half_rn(v.x)), __half2float(__float2half_rn(v.y)));
    b = make_float2(__half2float(__float2half_rn(v.z)), __half2float(__float2half_rn(v.w)));
  } else {
    const uint2 u = *reinterpret_cast<const uint2*>(x + (size_t)row * kHidden + c);
    a = __half22float2(u32_as_half2(u.x));
    b = __half22float2(u32_as_half2(u.y));
  }
  if (res != nullptr) {
    const float2 ra = __half22float2(u32_as_half2(r.x)), rb = __half22float2(u32_as_half2(r.y));
    // the residual stream is an fp16 tensor: round the sum
    a.x = __half2float(__float2half_rn(a.x + ra.x));
    a.y = __half2float(__float2half_rn(a.y + ra.y));
    b.x = __half2float(__float2half_rn(b.x + rb.x));
    b.y = __half2float(__float2half_rn(b.y + rb.y));
    if (sum_out != nullptr) {
      half2 o0 = __floats2half2_rn(a.x, a.y), o1 = __floats2half2_rn(b.x, b.y);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&o0);
      o.y = *reinterpret_cast<uint32_t*>(&o1);
      *reinterpret_cast<uint2*>(sum_out + (size_t)row * kHidden + c) = o;
    }
  }
  float ssq = warp_sum(a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y);
  if ((t & 31) == 0) red[t >> 5] = ssq;
  __syncthreads();
  ssq = 0.f;
#pragma unroll
  for (int i = 0; i < 7; ++i) ssq += red[i];
  const float rs = rsqrtf(ssq * (1.0f / kHidden) + eps);
  const float2 wa = __half22float2(u32_as_half2(wv.x)), wb = __half22float2(u32_as_half2(wv.y));
  half2 o0 = __floats2half2_rn(a.x * rs * wa.x, a.y * rs * wa.y);
  half2 o1 = __floats2half2_rn(b.x * rs * wb.x, b.y * rs * wb.y);
  uint2 o;
  o.x = *reinterpret_cast<uint32_t*>(&o0);
  o.y = *reinterpret_cast<uint32_t*>(&o1);
  *reinterpret_cast<uint2*>(y + (size_t)row * kHidden + c) = o;
}

// ---- RoPE --------------------------------------------------------------------
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, half* __restrict__ cos_t,
                                  half* __restrict__ sin_t, int max_pos) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= max_pos * 32) return;
  const int t = idx >> 5, c = idx & 31;
  const float ang = (float)t * inv_freq[c];
  float s, co;
  sincosf(ang, &s, &co);  // accurate range reduction (no fast-math in this file)
  cos_t[idx] = __float2half_rn(co);
  sin_t[idx] = __float2half_rn(s);
}

// x [B,H,S,64]; one thread per (b,h,s,pair).
__global__ void rope_kernel(const half* __restrict__ x, const half* __restrict__ cos_t,
                            const half* __restrict__ sin_t, half* __restrict__ y, int B, int H,
                            int S, int trig_batch_stride) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)B * H * S * 32;
  if (idx >= total) return;
  const int pair = idx & 31;
  const size_t vec = idx >> 5;  // (b,h,s)
  const int s = vec % S;
  const int b = vec / ((size_t)H * S);
  const size_t trig = (size_t)b * trig_batch_stride + (size_t)s * 32 + pair;
  const float c = __half2float(cos_t[trig]), sn = __half2float(sin_t[trig]);
  const float v0 = __half2float(x[vec * 64 + pair]);
  const float v1 = __half2float(x[vec * 64 + pair + 32]);
  y[vec * 64 + pair] = __float2half_rn(v0 * c - v1 * sn);
  y[vec * 64 + pair + 32] = __float2half_rn(v0 * sn + v1 * c);
}

// ---- SwiGLU -------------------------------------------------------------------
__global__ void swiglu_kernel(const half2* __restrict__ g, const half2* __restrict__ u,
                              half2* __restrict__ y, size_t n2) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n2) return;
  const float2 a = __half22float2(g[i]), b = __half22float2(u[i]);
  y[i] = __floats2half2_rn(silu_mul(a.x, b.x), silu_mul(a.y, b.y));
}

// ---- argmax --------------------------------------------------------------------
// One CTA per row; 16-byte loads when the row start is aligned.
__global__ void __launch_bounds__(1024) argmax_kernel(const half* __restrict__ logits, int V,
                                                      int64_t* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const half* row = logits + (size_t)blockIdx.x * V;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = __half2float(row[i]);
    if (v > bv) {  // ascending scan per thread: first maximum kept
      bv = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) {
      bv = ov;
      bi = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sv[warp] = bv;
    si[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    bv = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
  }
}

// ---- fp16 GEMV: y[m,n] = sum_k x[m,k] w[n,k] (+bias) ---------------------------
// One warp per output row n, up to 8 batch rows per pass, K multiple of 8.
template <int M>
__global__ void __launch_bounds__(256) gemv_f16_kernel(const half* __restrict__ x,
                                                       const half* __restrict__ w,
                                                       const half* __restrict__ bias,
                                                       half* __restrict__ y, int m_total, int N,
                                                       int K) {
  const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int row0 = blockIdx.y * M;
  if (n >= N) return;
  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  const uint4* wr = reinterpret_cast<const uint4*>(w + (size_t)n * K);
  for (int c = lane; c < K / 8; c += 32) {
    const uint4 wv = ldg_nc_u128(wr + c);
    const half2* wh = reinterpret_cast<const half2*>(&wv);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      if (row0 + m >= m_total) continue;
      const uint4 xv = *reinterpret_cast<const uint4*>(x + (size_t)(row0 + m) * K + 8 * c);
      const half2* xh = reinterpret_cast<const half2*>(&xv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 a = __half22float2(wh[e]), b = __half22float2(xh[e]);
        acc[m] = fmaf(a.x, b.x, acc[m]);
        acc[m] = fmaf(a.y, b.y, acc[m]);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const float s = warp_sum(acc[m]);
    if (lane == 0 && row0 + m < m_total) {
      float v = s;
      if (bias != nullptr) v = __half2float(__float2half_rn(v)) + __half2float(bias[n]);
      y[(size_t)(row0 + m) * N + n] = __float2half_rn(v);
    }
  }
}

// ---- pieces of the batched (batch > 8) decode step ------------------------------
// Embedding rows of the tokens the slots feed next: x[b] = embed[tok[rows[b]]].
__global__ void embed_rows_kernel(const half* __restrict__ embed, const int32_t* __restrict__ rows,
                                  const int32_t* __restrict__ tok, int vocab, half* __restrict__ x, int batch) {
  const int b = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (b >= batch) return;
  int t = tok[rows[b]];
  t = t < 0 ? 0 : (t >= vocab ? vocab - 1 : t);
  const uint2* src = reinterpret_cast<const uint2*>(embed + (size_t)t * kHidden);
  uint2* dst = reinterpret_cast<uint2*>(x + (size_t)b * kHidden);
  for (int i = threadIdx.x; i < kHidden / 4; i += blockDim.x) dst[i] = src[i];
}

// RoPE + q buffer + KV append from the fused QKV output (columns in rope-pair order,
// bias already added).  One thread per (row, column pair).
__global__ void qkv_post_kernel(const half* __restrict__ qkv, const float* __restrict__ part, int splits,
                                const half* __restrict__ bias, const int32_t* __restrict__ rows,
                                const int32_t* __restrict__ pos, const half* __restrict__ cos_t,
                                const half* __restrict__ sin_t, int max_pos, half* __restrict__ qbuf,
                                half* __restrict__ kcache, half* __restrict__ vcache, int s_max, int batch,
                                const int32_t* __restrict__ row_pos, int q_head_major, int n_slots) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (idx >= batch * (kQkvN / 2)) return;
  const int b = idx / (kQkvN / 2), c2 = idx % (kQkvN / 2);
  const int head = c2 >> 5, pair = c2 & 31;  // stored columns (2*pair, 2*pair+1) = dims (pair, pair+32)
  const int slot = rows[b];
  const bool slot_ok = slot >= 0 && slot < n_slots;  // a row with a slot outside the cache appends nothing
  // decode: the row's position is its slot's; prefill: every row (token) brings its own
  const int p = row_pos != nullptr ? row_pos[b] : (slot_ok ? pos[slot] : 0);
  float2 v;
  if (part != nullptr) {  // fp16(sum of the split-K partials) + bias, as the GEMM epilogue would do
    float2 p[16];
#pragma unroll
    for (int s = 0; s < 16; ++s)
      p[s] = s < splits ? __ldcg(reinterpret_cast<const float2*>(part + ((size_t)s * batch + b) * kQkvN + 2 * c2))
                        : make_float2(0.f, 0.f);
    float2 acc = make_float2(0.f, 0.f);
#pragma unroll
    for (int s = 0; s < 16; ++s) {
      acc.x += p[s].x;
      acc.y += p[s].y;
    }
    const float2 bb = __half22float2(*reinterpret_cast<const half2*>(bias + 2 * c2));
    v.x = __half2float(__float2half_rn(__half2float(__float2half_rn(acc.x)) + bb.x));
    v.y = __half2float(__float2half_rn(__half2float(__float2half_rn(acc.y)) + bb.y));
  } else {
    v = __half22float2(*reinterpret_cast<const half2*>(qkv + (size_t)b * kQkvN + 2 * c2));
  }
  float lo = v.x, hi = v.y;
  if (head < kHeads + kKvHeads) {
    const int pp = p < max_pos ? (p < 0 ? 0 : p) : max_pos - 1;
    const float c = __half2float(cos_t[(size_t)pp * 32 + pair]), s = __half2float(sin_t[(size_t)pp * 32 + pair]);
    lo = v.x * c - v.y * s;
    hi = v.x * s + v.y * c;
  }
  half* dst;
  if (head < kHeads) {
    dst = q_head_major ? qbuf + ((size_t)head * batch + b) * kHeadDim : qbuf + ((size_t)b * kHeads + head) * kHeadDim;
  } else {
    if (p >= s_max || p < 0 || !slot_ok) return;
    const int kvh = (head - kHeads) & 1;
    half* base = (head < kHeads + kKvHeads) ? kcache : vcache;
    dst = base + (((size_t)slot * kKvHeads + kvh) * s_max + p) * kHeadDim;
  }
  dst[pair] = __float2half_rn(lo);
  dst[pair + 32] = __float2half_rn(hi);
}

// The same for many rows (prefill: every row brings its own slot and position, q is written
// head-major): one thread per (row, head, 8 of the 64 dims), which reads the 8 stored pairs
// its dims come from (32 bytes) with their cos / sin (16 bytes each) and writes 16 bytes.
__global__ void __launch_bounds__(256) qkv_rope_rows_kernel(
    const half* __restrict__ qkv, const int32_t* __restrict__ slots, const int32_t* __restrict__ row_pos,
    const half* __restrict__ cos_t, const half* __restrict__ sin_t, int max_pos, half* __restrict__ qbuf,
    half* __restrict__ kcache, half* __restrict__ vcache, int s_max, int rows, int n_slots) {
  constexpr int kPerRow = (kHeads + 2 * kKvHeads) * 8;  // 144 threads per row
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (idx >= (size_t)rows * kPerRow) return;
  const int b = (int)(idx / kPerRow), rem = (int)(idx % kPerRow);
  const int head = rem >> 3, piece = rem & 7;   // piece: dims 8 piece .. 8 piece + 7
  const int pair0 = (piece & 3) * 8;            // their pairs: dims d and d + 32 are stored side by side
  const bool high = piece >= 4;                 // dims 32..63: the second element of the rotated pair
  const int slot = slots[b], p = row_pos[b];
  const half2* src = reinterpret_cast<const half2*>(qkv + (size_t)b * kQkvN + head * kHeadDim) + pair0;
  const uint4 in0 = *reinterpret_cast<const uint4*>(src), in1 = *reinterpret_cast<const uint4*>(src + 4);
  const half2 xy[8] = {*reinterpret_cast<const half2*>(&in0.x), *reinterpret_cast<const half2*>(&in0.y),
                       *reinterpret_cast<const half2*>(&in0.z), *reinterpret_cast<const half2*>(&in0.w),
                       *reinterpret_cast<const half2*>(&in1.x), *reinterpret_cast<const half2*>(&in1.y),
                       *reinterpret_cast<const half2*>(&in1.z), *reinterpret_cast<const half2*>(&in1.w)};
  half out[8];
  if (head < kHeads + kKvHeads) {
    const int pp = p < max_pos ? (p < 0 ? 0 : p) : max_pos - 1;
    const uint4 c4 = *reinterpret_cast<const uint4*>(cos_t + (size_t)pp * 32 + pair0);
    const uint4 s4 = *reinterpret_cast<const uint4*>(sin_t + (size_t)pp * 32 + pair0);
    const half* ch = reinterpret_cast<const half*>(&c4);
    const half* sh = reinterpret_cast<const half*>(&s4);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 v = __half22float2(xy[i]);
      const float c = __half2float(ch[i]), sn = __half2float(sh[i]);
      out[i] = __float2half_rn(high ? v.x * sn + v.y * c : v.x * c - v.y * sn);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = high ? __high2half(xy[i]) : __low2half(xy[i]);
  }
  half* dst;
  if (head < kHeads) {
    dst = qbuf + ((size_t)head * rows + b) * kHeadDim;
  } else {
    if (p >= s_max || p < 0 || slot < 0 || slot >= n_slots) return;  // nothing is appended for such a row
    const int kvh = (head - kHeads) & 1;
    half* base = (head < kHeads + kKvHeads) ? kcache : vcache;
    dst = base + (((size_t)slot * kKvHeads + kvh) * s_max + p) * kHeadDim;
  }
  *reinterpret_cast<uint4*>(dst + piece * 8) = *reinterpret_cast<const uint4*>(out);
}

// act[b][i] = silu(gu[b][i]) * gu[b][4864 + i] on the fused gate|up output, which comes
// either as fp16 rows or as `splits` fp32 split-K partial sums [splits][batch][9728]; the
// summed linear output is rounded to fp16 first, as the un-split epilogue does.
__global__ void swiglu_fused_kernel(const half* __restrict__ gu, const float* __restrict__ part, int splits,
                                    half* __restrict__ act, int batch) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (idx >= (size_t)batch * (kInter / 2)) return;
  const int b = idx / (kInter / 2), i2 = idx % (kInter / 2);
  float2 g, u;
  if (part != nullptr) {
    const size_t plane = (size_t)batch * 2 * kInter;
    const float* row = part + (size_t)b * 2 * kInter;
    float2 gs[16], us[16];
#pragma unroll
    for (int s = 0; s < 16; ++s) {
      gs[s] = s < splits ? __ldcg(reinterpret_cast<const float2*>(row + s * plane) + i2) : make_float2(0.f, 0.f);
      us[s] = s < splits ? __ldcg(reinterpret_cast<const float2*>(row + s * plane + kInter) + i2)
                         : make_float2(0.f, 0.f);
    }
    g = gs[0];
    u = us[0];
#pragma unroll
    for (int s = 1; s < 16; ++s) {
      g.x += gs[s].x;
      g.y += gs[s].y;
      u.x += us[s].x;
      u.y += us[s].y;
    }
    g = __half22float2(__floats2half2_rn(g.x, g.y));
    u = __half22float2(__floats2half2_rn(u.x, u.y));
  } else {
    const half2* row = reinterpret_cast<const half2*>(gu + (size_t)b * 2 * kInter);
    g = __half22float2(row[i2]);
    u = __half22float2(row[kInter / 2 + i2]);
  }
  reinterpret_cast<half2*>(act + (size_t)b * kInter)[i2] = __floats2half2_rn(silu_mul(g.x, u.x), silu_mul(g.y, u.y));
}

}  // namespace

cudaError_t launch_embed_rows(const half* embed, const int32_t* rows, const int32_t* tok, int vocab, half* x,
                              int batch, cudaStream_t st, bool pdl) {
  return launch(embed_rows_kernel, dim3(batch), dim3(224), 0, st, pdl, embed, rows, tok, vocab, x, batch);
}
cudaError_t launch_qkv_post(const half* qkv, const int32_t* rows, const int32_t* pos, const half* cos_t,
                            const half* sin_t, int max_pos, half* qbuf, half* kcache, half* vcache, int s_max,
                            int n_slots, int batch, cudaStream_t st) {
  const int total = batch * (kQkvN / 2);
  return launch(qkv_post_kernel, dim3((total + 255) / 256), dim3(256), 0, st, true, qkv, (const float*)nullptr, 0,
                (const half*)nullptr, rows, pos, cos_t, sin_t, max_pos, qbuf, kcache, vcache, s_max, batch,
                (const int32_t*)nullptr, 0, n_slots);
}
cudaError_t launch_qkv_rope_append(const half* qkv, const int32_t* slots, const int32_t* positions, const half* cos_t,
                                   const half* sin_t, int max_pos, half* q_out, half* kcache, half* vcache, int s_max,
                                   int n_slots, int rows, cudaStream_t st, bool pdl) {
  const size_t total = (size_t)rows * (kHeads + 2 * kKvHeads) * 8;
  return launch(qkv_rope_rows_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, pdl, qkv, slots, positions,
                cos_t, sin_t, max_pos, q_out, kcache, vcache, s_max, rows, n_slots);
}
cudaError_t launch_qkv_post_part(const float* part, int splits, const half* bias, const int32_t* rows,
                                 const int32_t* pos, const half* cos_t, const half* sin_t, int max_pos, half* qbuf,
                                 half* kcache, half* vcache, int s_max, int n_slots, int batch, cudaStream_t st) {
  const int total = batch * (kQkvN / 2);
  return launch(qkv_post_kernel, dim3((total + 255) / 256), dim3(256), 0, st, true, (const half*)nullptr, part,
                splits, bias, rows, pos, cos_t, sin_t, max_pos, qbuf, kcache, vcache, s_max, batch,
                (const int32_t*)nullptr, 0, n_slots);
}
cudaError_t launch_rmsnorm_part(const float* part, int splits, const half* residual, const half* w, float eps,
                                half* y, half* sum_out, int rows, cudaStream_t st) {
  return launch(rmsnorm_kernel, dim3(rows), dim3(224), 0, st, true, (const half*)nullptr, part, splits, residual, w,
                eps, y, sum_out, rows);
}
cudaError_t launch_swiglu_fused(const half* gu, half* act, int batch, cudaStream_t st) {
  const size_t total = (size_t)batch * (kInter / 2);
  return launch(swiglu_fused_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, true, gu,
                (const float*)nullptr, 0, act, batch);
}
cudaError_t launch_rmsnorm(const half* x, const half* residual, const half* w, float eps, half* y, half* sum_out,
                           int rows, cudaStream_t st) {
  return launch(rmsnorm_kernel, dim3(rows), dim3(224), 0, st, true, x, (const float*)nullptr, 0, residual, w, eps, y,
                sum_out, rows);
}
}  // namespace quic

using namespace quic;

extern "C" const char* quic_last_error(void) { return g_err; }
extern "C" int quic_abi_version(void) { return 1; }
extern "C" void quic_set_pdl(int enabled) { quic::set_pdl(enabled != 0); }

extern "C" int quic_rmsnorm(const void* x, const void* residual, const void* w, float eps, void* y,
                            void* sum_out, int32_t rows, void* stream) {
  QUIC_REQUIRE(x && w && y, QUIC_E_ARG, "rmsnorm: null tensor");
  QUIC_REQUIRE(rows >= 0, QUIC_E_SHAPE, "rmsnorm: negative rows");
  QUIC_REQUIRE(((uintptr_t)x | (uintptr_t)w | (uintptr_t)y | (uintptr_t)residual |
                (uintptr_t)sum_out) % 8 == 0,
               QUIC_E_ARG, "rmsnorm: tensors must be 8-byte aligned");
  if (rows == 0) return QUIC_OK;
  rmsnorm_kernel<<<rows, 224, 0, (cudaStream_t)stream>>>(
      (const half*)x, nullptr, 0, (const half*)residual, (const half*)w, eps, (half*)y, (half*)sum_out, rows);
  QUIC_CUDA(cudaGetLastError());
  return QUIC_OK;
}

extern "C" int quic_rope_table_init(const float* inv_freq32, int32_t max_pos, void* cos_t,
                                    void* sin_t, void* stream) {
  QUIC_REQUIRE(inv_freq32 && cos_t && sin_t, QUIC_E_ARG, "rope_table_init: null tensor");
  QUIC_REQUIRE(max_pos >= 1, QUIC_E_SHAPE, "rope_table_init: max_pos < 1");
  const int total = max_pos * 32;
  rope_table_kernel<<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
      inv_freq32, (half*)cos_t, (half*)sin_t, max_pos);
  QUIC_CUDA(cudaGetLastError());
  return QUIC_OK;
}

extern "C" int quic_rope(const void* x, const void* cos_t, const void* sin_t, void* y, int32_t b,
                         int32_t h, int32_t s, int32_t trig_batch_stride, void* stream) {
  QUIC_REQUIRE(x && cos_t && sin_t && y, QUIC_E_ARG, "rope: null tensor");
  QUIC_REQUIRE(b >= 0 && h >= 0 && s >= 0, QUIC_E_SHAPE, "rope: negative size");
  const size_t total = (size_t)b * h * s * 32;
  if (total == 0) return QUIC_OK;
  rope_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const half*)x, (const half*)cos_t, (const half*)sin_t, (half*)y, b, h, s, trig_batch_stride);
  QUIC_CUDA(cudaGetLastError());
  return QUIC_OK;
}

extern "C" int quic_swiglu(const void* gate, const void* up, void* y, int32_t rows, void* stream) {
  QUIC_REQUIRE(gate && up && y, QUIC_E_ARG, "swiglu: null tensor");
  QUIC_REQUIRE(rows >= 0, QUIC_E_SHAPE, "swiglu: negative rows");
  const size_t n2 = (size_t)rows * kInter / 2;
  if (n2 == 0) return QUIC_OK;
  swiglu_kernel<<<(unsigned)((n2 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const half2*)gate, (const half2*)up, (half2*)y, n2);
  QUIC_CUDA(cudaGetLastError());
  return QUIC_OK;
}

extern "C" int quic_qkv_rope_append(const void* qkv, const int32_t* slots, const int32_t* positions,
                                    const void* cos_t, const void* sin_t, int32_t max_pos, void* q_out,
                                    void* kcache, void* vcache, int32_t s_max, int32_t n_slots, int32_t rows,
                                    void* stream) {
  QUIC_REQUIRE(qkv && slots && positions && cos_t && sin_t && q_out && kcache && vcache, QUIC_E_ARG,
               "qkv_rope_append: null tensor");
  QUIC_REQUIRE(rows >= 0 && rows <= (1 << 20) && s_max >= 1 && max_pos >= 1 && n_slots >= 1, QUIC_E_SHAPE,
               "qkv_rope_append: bad row count or cache geometry");
  QUIC_REQUIRE(((uintptr_t)qkv | (uintptr_t)cos_t | (uintptr_t)sin_t | (uintptr_t)q_out | (uintptr_t)kcache |
                (uintptr_t)vcache) % 16 == 0,
               QUIC_E_ARG, "qkv_rope_append: tensors must be 16-byte aligned");
  if (rows == 0) return QUIC_OK;
  QUIC_CUDA(launch_qkv_rope_append((const half*)qkv, slots, positions, (const half*)cos_t, (const half*)sin_t,
                                   (int)max_pos, (half*)q_out, (half*)kcache, (half*)vcache, (int)s_max, (int)n_slots,
                                   (int)rows, (cudaStream_t)stream, false));
  return QUIC_OK;
}

extern "C" int quic_swiglu_fused(const void* gu, void* y, int32_t rows, void* stream) {
  QUIC_REQUIRE(gu && y, QUIC_E_ARG, "swiglu_fused: null tensor");
  QUIC_REQUIRE(rows >= 0, QUIC_E_SHAPE, "swiglu_fused: negative rows");
  if (rows == 0) return QUIC_OK;
  const size_t total = (size_t)rows * (kInter / 2);
  QUIC_CUDA(launch(swiglu_fused_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
                   false, (const half*)gu, (const float*)nullptr, 0, (half*)y, (int)rows));
  return QUIC_OK;
}

extern "C" int quic_argmax(const void* logits, int32_t b, int32_t v, int64_t* out, void* stream) {
  QUIC_REQUIRE(logits && out, QUIC_E_ARG, "argmax: null tensor");
  QUIC_REQUIRE(b >= 0 && v >= 1, QUIC_E_SHAPE, "argmax: bad shape");
  if (b == 0) return QUIC_OK;
  argmax_kernel<<<b, 1024, 0, (cudaStream_t)stream>>>((const half*)logits, v, out);
  QUIC_CUDA(cudaGetLastError());
  return QUIC_OK;
}

extern "C" int quic_gemm_f16(const void* x, const void* w, const void* bias, void* y, int32_t m,
                             int32_t n, int32_t k, void* stream) {
  QUIC_REQUIRE(x && w && y, QUIC_E_ARG, "gemm_f16: null tensor");
  QUIC_REQUIRE(m >= 0 && n >= 1 && k >= 8 && k % 8 == 0, QUIC_E_SHAPE,
               "gemm_f16: K must be a positive multiple of 8");
  QUIC_REQUIRE(((uintptr_t)x | (uintptr_t)w) % 16 == 0, QUIC_E_ARG,
               "gemm_f16: x and w must be 16-byte aligned");
  if (m == 0) return QUIC_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int mchunks = (m + 7) / 8;
  QUIC_REQUIRE(mchunks <= 65535, QUIC_E_SHAPE, "gemm_f16: too many rows");
  dim3 grid((n + 7) / 8, mchunks);
  if (m == 1)
    gemv_f16_kernel<1><<<grid, 256, 0, st>>>((const half*)x, (const half*)w, (const half*)bias,
                                             (half*)y, m, n, k);
  else
    gemv_f16_kernel<8><<<grid, 256, 0, st>>>((const half*)x, (const half*)w, (const half*)bias,
                                             (half*)y, m, n, k);
  QUIC_CUDA(cudaGetLastError());
  return QUIC_OK;
}


