// The four linears of a decoder layer with DENSE fp16 weights for one or two batch rows: the
// un-quantised model through the same fused decode step (the reference's second execution
// path: src/model.py:35-41 falls to kernels/cuda/gemm.cu:36 when a linear carries no packed
// weight).  Same fusion as the W4A16 chain -- RMSNorm in front, bias / RoPE / KV append,
// residual add and SwiGLU behind -- around a GEMV over weights stored [N, K] with K
// contiguous (the checkpoint's own layout; q|k|v and gate|up fused along N, the q and k rows
// of a head in rotation-pair order).
//
// Shape of every kernel: a warp per output column (two weight rows for gate|up; four warps per
// column, a quarter of K each, for down), lanes striding K in 16-byte pieces, the M activation
// rows in shared memory, fp32 accumulation with mixed-precision FMAs.  The weights are four
// times the int4 ones (29.8 MB per layer), so these kernels are bound by streaming them: every
// lane requests ALL its weight pieces (at most five) before griddepcontrol.wait, so the whole
// matrix is in flight while the previous kernel of the chain still runs, and after the wait
// only the activations are fetched.  No cross-CTA reduction: a column is finished by its CTA.
//
// Rounding points as in the W4A16 chain (decode_layers.cu): a linear's output is an fp16
// tensor, so is the residual stream, the normalised activation and the SwiGLU output.
#include "decode_kernels.cuh"

namespace quic {
namespace {

constexpr int kF16Warps = 8;
constexpr int kF16Threads = kF16Warps * 32;

// acc += dot of 8 fp16 weights with 8 fp16 activations: mixed-precision FMA (fp16 operands, fp32
// accumulator, no conversions), two accumulators so that consecutive FMAs are independent.
__device__ __forceinline__ void dot8(const uint4& w, const uint4& x, float (&acc)[2]) {
  const half2* wh = reinterpret_cast<const half2*>(&w);
  const half2* xh = reinterpret_cast<const half2*>(&x);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[0] = fma_h(acc[0], __low2half(wh[i]), __low2half(xh[i]));
    acc[1] = fma_h(acc[1], __high2half(wh[i]), __high2half(xh[i]));
  }
}

// The lane's pieces (16 bytes each, lane + 32 u) of `nvec` pieces of a weight row, all requested
// at once: ceil(nvec / 32) <= kMaxPieces loads in flight per lane.
constexpr int kMaxPieces = 5;
struct RowRegs {
  uint4 w[kMaxPieces];
};
__device__ __forceinline__ void load_row(RowRegs& r, const half* wrow, int nvec, int lane) {
  const uint4* wp = reinterpret_cast<const uint4*>(wrow);
#pragma unroll
  for (int u = 0; u < kMaxPieces; ++u) {
    const int i = lane + 32 * u;
    r.w[u] = make_uint4(0u, 0u, 0u, 0u);
    if (i < nvec) r.w[u] = ldg_nc_u128(wp + i);
  }
}
// acc[m] = sum over the lane's pieces of W . xs[m] (xs: the M rows, `stride` halves apart, at the
// row's first k); the warp total is on every lane on return.
template <int M>
__device__ __forceinline__ void row_dot(const RowRegs& r, const half* xs, int stride, int nvec, int lane,
                                        float (&acc)[M]) {
  float a2[M][2];
#pragma unroll
  for (int m = 0; m < M; ++m) a2[m][0] = a2[m][1] = 0.f;
#pragma unroll
  for (int u = 0; u < kMaxPieces; ++u) {
    const int i = lane + 32 * u;
    if (i < nvec) {
#pragma unroll
      for (int m = 0; m < M; ++m) dot8(r.w[u], *reinterpret_cast<const uint4*>(xs + (size_t)m * stride + 8 * i), a2[m]);
    }
  }
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = warp_sum(a2[m][0] + a2[m][1]);
}

// M rows of 896 halves -> xs, RMS-normalised when ln != nullptr (fp32 statistics, fp16 result,
// as the reference's rmsnorm kernel).  src[m] == nullptr: a row beyond the batch, zeros.
// red: [M][8] floats.  256 threads; ends with a CTA barrier.
template <int M>
__device__ __forceinline__ void stage_hidden(half* xs, float* red, const half* const (&src)[M], const half* ln,
                                             float eps, half* raw_out, int row0) {
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  uint4 v[M];
  float ss[M];
#pragma unroll
  for (int m = 0; m < M; ++m) {
    v[m] = make_uint4(0u, 0u, 0u, 0u);
    ss[m] = 0.f;
    if (t < kHidden / 8 && src[m] != nullptr) {
      v[m] = __ldcg(reinterpret_cast<const uint4*>(src[m]) + t);
      if (raw_out != nullptr) reinterpret_cast<uint4*>(raw_out + (size_t)(row0 + m) * kHidden)[t] = v[m];
      const half2* h = reinterpret_cast<const half2*>(&v[m]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h[e]);
        ss[m] += f.x * f.x + f.y * f.y;
      }
    }
  }
  if (ln != nullptr) {
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const float s = warp_sum(ss[m]);
      if (lane == 0) red[m * kF16Warps + warp] = s;
    }
    __syncthreads();
  }
  if (t < kHidden / 8) {
    uint4 wv = make_uint4(0u, 0u, 0u, 0u);
    if (ln != nullptr) wv = ldg_nc_u128(reinterpret_cast<const uint4*>(ln) + t);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      uint4 o = v[m];
      if (ln != nullptr) {
        float ssq = 0.f;
#pragma unroll
        for (int w = 0; w < kF16Warps; ++w) ssq += red[m * kF16Warps + w];
        const float r = rsqrtf(ssq * (1.0f / kHidden) + eps);
        const half2* h = reinterpret_cast<const half2*>(&v[m]);
        const half2* w2 = reinterpret_cast<const half2*>(&wv);
        half2* oh = reinterpret_cast<half2*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __half22float2(h[e]), wf = __half22float2(w2[e]);
          oh[e] = __floats2half2_rn(f.x * r * wf.x, f.y * r * wf.y);
        }
      }
      reinterpret_cast<uint4*>(xs + (size_t)m * kHidden)[t] = o;
    }
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------
// K1: (embedding gather |) RMSNorm -> QKV -> bias -> RoPE -> q buffer / KV append.
// grid (144, ceil(batch / M)): 8 columns per CTA, i.e. four rotation pairs.
// ---------------------------------------------------------------------------
struct QkvF16Args {
  const half* w;     // [1152][896], rows of a head in rotation-pair order
  const half* bias;  // [1152] same order, or nullptr
  const half* ln;
  const half* embed;
  const half* x_in;  // [batch][896]
  half* x_copy;      // first layer: the gathered rows (the layer's residual input)
  RowState rs;
  float eps;
  int32_t first_layer, vocab;
  const half* cos_t;
  const half* sin_t;
  int32_t max_pos;
  half* qbuf;
  half* kcache;
  half* vcache;
  int32_t s_max, n_slots;
};

template <int M>
__global__ void __launch_bounds__(kF16Threads) qkv_f16_kernel(const QkvF16Args a) {
  __shared__ __align__(16) half xs[M * kHidden];
  __shared__ float red[M * kF16Warps];
  __shared__ float vals[kF16Warps][M];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * kF16Warps + warp;
  const int row0 = blockIdx.y * M;
  const half* wrow = a.w + (size_t)n * kHidden;
  pdl_trigger_early();
  RowRegs wr;
  load_row(wr, wrow, kHidden / 8, lane);  // weights: not written by the chain, requested before the wait
  const float bias = a.bias != nullptr ? __half2float(a.bias[n]) : 0.f;
  int slot[M];
#pragma unroll
  for (int m = 0; m < M; ++m) slot[m] = (row0 + m < a.rs.batch) ? a.rs.rows[row0 + m] : -1;
  pdl_wait();

  const half* src[M];
  int pos[M];
#pragma unroll
  for (int m = 0; m < M; ++m) {
    src[m] = nullptr;
    pos[m] = 0;
    if (slot[m] >= 0 && slot[m] < a.n_slots) {
      pos[m] = __ldcg(a.rs.pos + slot[m]);
      if (a.first_layer) {
        int tk = __ldcg(a.rs.tok + slot[m]);
        tk = tk < 0 ? 0 : (tk >= a.vocab ? a.vocab - 1 : tk);
        src[m] = a.embed + (size_t)tk * kHidden;
      } else {
        src[m] = a.x_in + (size_t)(row0 + m) * kHidden;
      }
    }
  }
  stage_hidden<M>(xs, red, src, a.ln, a.eps, (a.first_layer && blockIdx.x == 0) ? a.x_copy : nullptr, row0);

  float acc[M];
  row_dot<M>(wr, xs, kHidden, kHidden / 8, lane, acc);
  pdl_trigger_late();
  if (lane == 0) {
#pragma unroll
    for (int m = 0; m < M; ++m)  // fp16 linear output with bias, as the reference's GEMM writes it
      vals[warp][m] = __half2float(__float2half_rn(__half2float(__float2half_rn(acc[m])) + bias));
  }
  __syncthreads();

  // epilogue: thread -> (row m, rotation pair p of the CTA's four)
  if (threadIdx.x < M * 4) {
    const int m = threadIdx.x >> 2, p = threadIdx.x & 3;
    const int col = blockIdx.x * kF16Warps + 2 * p;  // stored columns (col, col + 1) = dims (pj, pj + 32)
    const int head = col >> 6, pj = (col & 63) >> 1;
    int sl = -1, ps = 0;
#pragma unroll
    for (int mm = 0; mm < M; ++mm)
      if (mm == m) { sl = slot[mm]; ps = pos[mm]; }
    if (sl >= 0 && sl < a.n_slots) {
      const float v0 = vals[2 * p][m], v1 = vals[2 * p + 1][m];
      float lo = v0, hi = v1;
      if (head < kHeads + kKvHeads) {
        const int pc = ps < a.max_pos ? (ps < 0 ? 0 : ps) : a.max_pos - 1;
        const float cs = __half2float(a.cos_t[(size_t)pc * 32 + pj]), sn = __half2float(a.sin_t[(size_t)pc * 32 + pj]);
        lo = v0 * cs - v1 * sn;
        hi = v0 * sn + v1 * cs;
      }
      const half lo16 = __float2half_rn(lo), hi16 = __float2half_rn(hi);
      if (head < kHeads) {
        half* q = a.qbuf + ((size_t)(row0 + m) * kHeads + head) * kHeadDim;
        q[pj] = lo16;
        q[pj + 32] = hi16;
      } else if (ps >= 0 && ps < a.s_max) {
        const int kvh = (head - kHeads) & 1;
        half* base = head < kHeads + kKvHeads ? a.kcache : a.vcache;
        half* dst = base + (((size_t)sl * kKvHeads + kvh) * a.s_max + ps) * kHeadDim;
        dst[pj] = lo16;
        dst[pj + 32] = hi16;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// K3: o_proj -> residual add.  grid (112, ceil(batch / M)).
// K5: down -> residual add (K = 4864).  Same kernel, the activation rows in dynamic shared memory.
// ---------------------------------------------------------------------------
struct ResidualF16Args {
  const half* w;        // [896][K]
  const half* x;        // [batch][K] the linear's input
  const half* xres_in;  // [batch][896]
  half* xres_out;
  int32_t batch, k;
};

// KW warps share a column, each owning a contiguous 1/KW of K (KW = 1 for o_proj, 4 for down, so
// that a lane holds at most kMaxPieces pieces and every weight byte of the kernel is requested
// at once); 8 columns per CTA, the KW partial sums of a column meet in shared memory.
template <int M, int KW>
__global__ void __launch_bounds__(kF16Threads * KW) residual_f16_kernel(const ResidualF16Args a) {
  extern __shared__ __align__(16) unsigned char smem_dyn[];
  half* xs = reinterpret_cast<half*>(smem_dyn);  // [M][K]
  __shared__ float part[KW][kF16Warps][M];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cw = warp % kF16Warps, kq = warp / kF16Warps;  // column of the CTA, quarter of K
  const int n = blockIdx.x * kF16Warps + cw;
  const int row0 = blockIdx.y * M;
  const int kpart = a.k / KW;  // multiple of 8
  const half* wrow = a.w + (size_t)n * a.k + (size_t)kq * kpart;
  pdl_trigger_early();
  RowRegs wr;
  load_row(wr, wrow, kpart / 8, lane);
  pdl_wait();

  const int nvec = a.k >> 3;
  for (int p = threadIdx.x; p < M * nvec; p += kF16Threads * KW) {
    const int m = p / nvec, c = p - m * nvec;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row0 + m < a.batch) v = __ldcg(reinterpret_cast<const uint4*>(a.x + (size_t)(row0 + m) * a.k) + c);
    reinterpret_cast<uint4*>(xs + (size_t)m * a.k)[c] = v;
  }
  __syncthreads();
  float acc[M];
  row_dot<M>(wr, xs + (size_t)kq * kpart, a.k, kpart / 8, lane, acc);
  pdl_trigger_late();
  if (KW > 1) {
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < M; ++m) part[kq][cw][m] = acc[m];
    }
    __syncthreads();
    if (kq != 0) return;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float v = 0.f;
#pragma unroll
      for (int q = 0; q < KW; ++q) v += part[q][cw][m];
      acc[m] = v;
    }
  }
  if (lane < M && row0 + lane < a.batch) {
    float v = 0.f;
#pragma unroll
    for (int m = 0; m < M; ++m)
      if (m == lane) v = acc[m];
    const size_t idx = (size_t)(row0 + lane) * kHidden + n;
    a.xres_out[idx] = __float2half_rn(__half2float(a.xres_in[idx]) + __half2float(__float2half_rn(v)));
  }
}

// ---------------------------------------------------------------------------
// K4: RMSNorm -> gate & up -> SwiGLU.  grid (608, ceil(batch / M)): warp w of CTA c owns gate
// row 8 c + w and the up row of the same index, so SwiGLU stays inside the warp.
// ---------------------------------------------------------------------------
struct GateUpF16Args {
  const half* w;  // [9728][896]: gate rows then up rows
  const half* ln;
  const half* xres;  // [batch][896]
  half* act;         // [batch][4864]
  int32_t batch;
  float eps;
};

template <int M>
__global__ void __launch_bounds__(kF16Threads) gateup_f16_kernel(const GateUpF16Args a) {
  __shared__ __align__(16) half xs[M * kHidden];
  __shared__ float red[M * kF16Warps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * kF16Warps + warp;
  const int row0 = blockIdx.y * M;
  const half* grow = a.w + (size_t)c * kHidden;
  const half* urow = a.w + (size_t)(kInter + c) * kHidden;
  pdl_trigger_early();
  RowRegs gr, ur;
  load_row(gr, grow, kHidden / 8, lane);
  load_row(ur, urow, kHidden / 8, lane);
  pdl_wait();

  const half* src[M];
#pragma unroll
  for (int m = 0; m < M; ++m) src[m] = row0 + m < a.batch ? a.xres + (size_t)(row0 + m) * kHidden : nullptr;
  stage_hidden<M>(xs, red, src, a.ln, a.eps, nullptr, row0);
  float g[M], u[M];
  row_dot<M>(gr, xs, kHidden, kHidden / 8, lane, g);
  row_dot<M>(ur, xs, kHidden, kHidden / 8, lane, u);
  pdl_trigger_late();
  if (lane < M && row0 + lane < a.batch) {
    float gv = 0.f, uv = 0.f;
#pragma unroll
    for (int m = 0; m < M; ++m)
      if (m == lane) { gv = g[m]; uv = u[m]; }
    // gate and up are fp16 linear outputs in the reference; the SwiGLU output is fp16 too
    a.act[(size_t)(row0 + lane) * kInter + c] =
        __float2half_rn(silu_mul(__half2float(__float2half_rn(gv)), __half2float(__float2half_rn(uv))));
  }
}

template <int M>
cudaError_t launch_residual(const ResidualF16Args& a, cudaStream_t st) {
  const size_t smem = (size_t)M * a.k * sizeof(half);  // at most 2 x 4864 x 2 = 19,456 bytes
  const dim3 grid(kHidden / kF16Warps, (a.batch + M - 1) / M);
  if (a.k == kInter) return launch(residual_f16_kernel<M, 4>, grid, dim3(kF16Threads * 4), smem, st, true, a);
  return launch(residual_f16_kernel<M, 1>, grid, dim3(kF16Threads), smem, st, true, a);
}

}  // namespace

#define QUIC_F16_DISPATCH_M(batch, fn, ...)    \
  do {                                         \
    if ((batch) <= 1) return fn<1>(__VA_ARGS__); \
    return fn<2>(__VA_ARGS__);                 \
  } while (0)

namespace {
template <int M>
cudaError_t launch_qkv_m(const QkvF16Args& a, cudaStream_t st, bool pdl) {
  return launch(qkv_f16_kernel<M>, dim3(kQkvN / kF16Warps, (a.rs.batch + M - 1) / M), dim3(kF16Threads), 0, st, pdl, a);
}
template <int M>
cudaError_t launch_gateup_m(const GateUpF16Args& a, cudaStream_t st) {
  return launch(gateup_f16_kernel<M>, dim3(kInter / kF16Warps, (a.batch + M - 1) / M), dim3(kF16Threads), 0, st, true, a);
}
}  // namespace

// Launchers of the dense chain (1..kF16ChainMaxRows rows per launch; more rows tile over grid.y).
cudaError_t launch_qkv_f16(const quic_w4_t& w, const half* ln, const half* embed, const half* x_in, half* x_copy,
                           const RowState& rs, float eps, bool first_layer, int vocab, const half* cos_t,
                           const half* sin_t, int max_pos, half* qbuf, half* kcache, half* vcache, int s_max,
                           int n_slots, cudaStream_t st, bool pdl) {
  QkvF16Args a = {};
  a.w = (const half*)w.w16;
  a.bias = (const half*)w.bias;
  a.ln = ln;
  a.embed = embed;
  a.x_in = x_in;
  a.x_copy = x_copy;
  a.rs = rs;
  a.eps = eps;
  a.first_layer = first_layer ? 1 : 0;
  a.vocab = vocab;
  a.cos_t = cos_t;
  a.sin_t = sin_t;
  a.max_pos = max_pos;
  a.qbuf = qbuf;
  a.kcache = kcache;
  a.vcache = vcache;
  a.s_max = s_max;
  a.n_slots = n_slots;
  QUIC_F16_DISPATCH_M(rs.batch, launch_qkv_m, a, st, pdl);
}

cudaError_t launch_residual_f16(const quic_w4_t& w, const half* x, const half* xres_in, half* xres_out, int batch,
                                cudaStream_t st) {
  ResidualF16Args a = {};
  a.w = (const half*)w.w16;
  a.x = x;
  a.xres_in = xres_in;
  a.xres_out = xres_out;
  a.batch = batch;
  a.k = w.k;
  QUIC_F16_DISPATCH_M(batch, launch_residual, a, st);
}

cudaError_t launch_gateup_f16(const quic_w4_t& w, const half* ln, const half* xres, half* act, int batch, float eps,
                              cudaStream_t st) {
  GateUpF16Args a = {};
  a.w = (const half*)w.w16;
  a.ln = ln;
  a.xres = xres;
  a.act = act;
  a.batch = batch;
  a.eps = eps;
  QUIC_F16_DISPATCH_M(batch, launch_gateup_m, a, st);
}

}  // namespace quic
