// W4A16 weights: checkpoint -> device layout repack, fp16 dequantisation (for
// bit-exactness checks) and the generic dequant-GEMV linear for any
// (N % 32 == 0, K % 128 == 0) and any row count.
#include "decode_kernels.cuh"

namespace quic {

namespace {

// Source row for stored row r of the layer (QUIC_ROWS_ROPE_PAIRS: stored
// (0,32,1,33,...) inside each block of 64).
__device__ __forceinline__ int src_row(int r, int order) {
  if (order == QUIC_ROWS_NATURAL) return r;
  const int i = r & 63;
  return (r & ~63) + (i >> 1) + 32 * (i & 1);
}

// One thread per (k-word j, stored row r) for the weights, and a strided tail
// for scales and zero points.
__global__ void prepack_kernel(const int32_t* __restrict__ packed, const half* __restrict__ scale,
                               const int32_t* __restrict__ zpw, int N, int K, int order,
                               int row_offset, int n_total, int32_t* __restrict__ qw,
                               half* __restrict__ sc, uint8_t* __restrict__ zp) {
  const int kw = K / 8, ng = K / kGroup;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < (size_t)kw * N) {
    const int j = idx / N, r = idx % N;
    const int n = src_row(r, order);
    qw[(size_t)j * n_total + row_offset + r] = packed[(size_t)n * kw + j];
  }
  if (idx < (size_t)ng * N) {
    const int g = idx / N, r = idx % N;
    const int n = src_row(r, order);
    sc[(size_t)g * n_total + row_offset + r] = scale[(size_t)n * ng + g];
  }
  if (idx < (size_t)ng * (N / 2)) {
    const int g = idx / (N / 2), r2 = idx % (N / 2);
    int byte = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = src_row(2 * r2 + h, order);
      // reference src/quant/checkpoint.py:31-32: row n -> word n/8, nibble n%8
      const int z = (zpw[(size_t)(n >> 3) * ng + g] >> (4 * (n & 7))) & 15;
      byte |= z << (4 * h);
    }
    zp[(size_t)g * (n_total / 2) + (row_offset / 2) + r2] = (uint8_t)byte;
  }
}

__global__ void dequant_kernel(const quic_w4_t w, half* __restrict__ out) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int kw = w.k / 8;
  if (idx >= (size_t)kw * w.n) return;
  const int j = idx / w.n, n = idx % w.n;
  const int g = (8 * j) / kGroup;
  const uint32_t word = (uint32_t)w.qw[(size_t)j * w.n + n];
  const half s = reinterpret_cast<const half*>(w.sc)[(size_t)g * w.n + n];
  const int z = (w.zp[(size_t)g * (w.n / 2) + (n >> 1)] >> (4 * (n & 1))) & 15;
  half2 d[4];
  dequant8(word, zp_to_half2(z), __half2half2(s), d);
  half* o = out + (size_t)n * w.k + 8 * j;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    o[p] = __low2half(d[p]);
    o[p + 4] = __high2half(d[p]);
  }
}

// Generic GEMV: CTA = 32 columns x (up to 16 warps striding the groups of its K
// split) x up to 8 batch rows; x is staged as fp16 in dynamic shared memory.
template <int M>
__global__ void __launch_bounds__(512) w4_gemv_kernel(const half* __restrict__ x, const quic_w4_t w,
                                                      half* __restrict__ y,
                                                      float* __restrict__ part, int m_total,
                                                      int groups_per_split) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  half* xs = reinterpret_cast<half*>(smem_raw);            // [M][kspan] perm8 order
  const int nwarp = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 32 + lane;
  const int ng = w.k / kGroup;
  const int g0 = blockIdx.y * groups_per_split;
  const int g1 = min(ng, g0 + groups_per_split);
  const int kspan = (g1 - g0) * kGroup;
  float* red = reinterpret_cast<float*>(smem_raw + (size_t)M * groups_per_split * kGroup * 2);
  const int row0 = blockIdx.z * M;

  for (int idx = threadIdx.x; idx < M * kspan; idx += blockDim.x) {
    const int m = idx / kspan, k = idx % kspan;
    half v = __float2half(0.f);
    if (row0 + m < m_total) v = x[(size_t)(row0 + m) * w.k + g0 * kGroup + k];
    xs[m * kspan + perm_k(k)] = v;
  }
  __syncthreads();

  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  const half* scp = reinterpret_cast<const half*>(w.sc);
  for (int g = g0 + warp; g < g1; g += nwarp) {
    const half2 s2 = __half2half2(scp[(size_t)g * w.n + n]);
    const half2 z2 =
        zp_to_half2((w.zp[(size_t)g * (w.n >> 1) + (n >> 1)] >> (4 * (n & 1))) & 15);
    uint32_t q[kWordsPerGroup];
#pragma unroll
    for (int j = 0; j < kWordsPerGroup; ++j)
      q[j] = ldg_nc_u32(w.qw + ((size_t)g * kWordsPerGroup + j) * w.n + n);
#pragma unroll
    for (int j = 0; j < kWordsPerGroup; ++j) {
      half2 d[4];
      dequant8(q[j], z2, s2, d);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const uint4 xv =
            *reinterpret_cast<const uint4*>(xs + m * kspan + (g - g0) * kGroup + 8 * j);
        const half2* xh = reinterpret_cast<const half2*>(&xv);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const float2 a = __half22float2(d[p]), b = __half22float2(xh[p]);
          acc[m] = fmaf(a.x, b.x, acc[m]);
          acc[m] = fmaf(a.y, b.y, acc[m]);
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < M; ++m) red[(warp * M + m) * 32 + lane] = acc[m];
  __syncthreads();
  for (int m = warp; m < M; m += nwarp) {
    if (row0 + m >= m_total) continue;
    float v = 0.f;
    for (int ww = 0; ww < nwarp; ++ww) v += red[(ww * M + m) * 32 + lane];
    if (gridDim.y == 1) {
      v = __half2float(__float2half_rn(v));
      if (w.bias) v += __half2float(reinterpret_cast<const half*>(w.bias)[n]);
      y[(size_t)(row0 + m) * w.n + n] = __float2half_rn(v);
    } else {
      part[((size_t)blockIdx.y * m_total + row0 + m) * w.n + n] = v;
    }
  }
}

__global__ void splitk_finish_kernel(const float* __restrict__ part, const half* __restrict__ bias,
                                     half* __restrict__ y, int m_total, int N, int splits) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)m_total * N) return;
  float v = 0.f;
  for (int s = 0; s < splits; ++s) v += part[(size_t)s * m_total * N + idx];
  v = __half2float(__float2half_rn(v));
  if (bias) v += __half2float(bias[idx % N]);
  y[idx] = __float2half_rn(v);
}

int gemv_splits(int n, int k) {
  // Aim at >= ~148 CTAs for one batch-row chunk.
  const int ng = k / kGroup;
  const int tiles = n / 32;
  int s = (148 + tiles - 1) / tiles;
  if (s > ng) s = ng;
  if (s < 1) s = 1;
  return s;
}

}  // namespace
}  // namespace quic

using namespace quic;

extern "C" int quic_w4_prepack(const int32_t* weight_packed, const void* weight_scale,
                               const int32_t* weight_zero_point, int32_t n, int32_t k,
                               int32_t row_order, int32_t row_offset, int32_t n_total, int32_t* qw,
                               void* sc, uint8_t* zp, void* stream) {
  QUIC_REQUIRE(weight_packed && weight_scale && weight_zero_point && qw && sc && zp, QUIC_E_ARG,
               "w4_prepack: null tensor");
  QUIC_REQUIRE(n > 0 && k > 0 && n % 32 == 0 && k % kGroup == 0, QUIC_E_SHAPE,
               "w4_prepack: N must be a multiple of 32 and K of 128");
  QUIC_REQUIRE(row_order == QUIC_ROWS_NATURAL || (row_order == QUIC_ROWS_ROPE_PAIRS && n % 64 == 0),
               QUIC_E_SHAPE, "w4_prepack: rope-pair order needs N multiple of 64");
  QUIC_REQUIRE(row_offset >= 0 && row_offset % 32 == 0 && row_offset + n <= n_total &&
                   n_total % 32 == 0,
               QUIC_E_SHAPE, "w4_prepack: bad row_offset / n_total");
  const size_t total = (size_t)(k / 8) * n;
  prepack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      weight_packed, (const half*)weight_scale, weight_zero_point, n, k, row_order, row_offset,
      n_total, qw, (half*)sc, zp);
  QUIC_CUDA(cudaGetLastError());
  return QUIC_OK;
}

extern "C" int quic_w4_dequant(const quic_w4_t* w, void* out, void* stream) {
  QUIC_REQUIRE(w && w->qw && w->sc && w->zp && out, QUIC_E_ARG, "w4_dequant: null tensor");
  QUIC_REQUIRE(w->n > 0 && w->k > 0 && w->n % 32 == 0 && w->k % kGroup == 0, QUIC_E_SHAPE,
               "w4_dequant: bad shape");
  const size_t total = (size_t)(w->k / 8) * w->n;
  dequant_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(*w, (half*)out);
  QUIC_CUDA(cudaGetLastError());
  return QUIC_OK;
}

// Rows from which the tcgen05 GEMM beats the dequant GEMV (measured per layer shape: 5-9 us
// against 10-19 us at 4 rows; the GEMV runs 2..8 rows on one 8-row instantiation).
static constexpr int kTensorMinRows = 2;

static int64_t packed_workspace_bytes(int32_t m, int32_t n, int32_t k);

extern "C" int64_t quic_w4a16_workspace_bytes(int32_t m, int32_t n, int32_t k) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  // the same block serves a packed or a dense weight of this shape
  const int64_t packed = packed_workspace_bytes(m, n, k), dense = gemm_f16_tc_workspace(m, n, k);
  return packed > dense ? packed : dense;
}

static int64_t packed_workspace_bytes(int32_t m, int32_t n, int32_t k) {
  // 16 KB reserved head, then split-K partials: of the tensor path from 2 rows (it stops
  // splitting once the output tiles fill the SMs, so large m needs none), of the GEMV below.
  if (m >= kTensorMinRows && n % 128 == 0 && k % 64 == 0) {
    const int64_t tc = 16384 + w4a16_gemm_tc_workspace(m, n, k);
    const int64_t gv = m > 8 ? 16384 + (int64_t)2 * m * n * 4 : 16384 + (int64_t)gemv_splits(n, k) * m * n * 4;
    return tc > gv ? tc : gv;  // the caller may force either path
  }
  if (m > 8) return 16384 + (int64_t)2 * m * n * 4;  // row-chunked GEMV splits only to fit shared memory
  return 16384 + (int64_t)gemv_splits(n, k) * m * n * 4;
}

extern "C" int quic_w4a16_linear(const void* x, const quic_w4_t* w, void* y, int32_t m,
                                 int32_t use_tensor, void* workspace, void* stream) {
  QUIC_REQUIRE(x && w && y, QUIC_E_ARG, "w4a16_linear: null tensor");
  if (w->w16 != nullptr) {  // dense fp16 weight [N, K]: a row or two on the GEMV, more on the tcgen05 GEMM
    QUIC_REQUIRE(w->n > 0 && w->k > 0 && w->k % 8 == 0 && m >= 0, QUIC_E_SHAPE, "linear: bad dense shape");
    if (m == 0) return QUIC_OK;
    if (m >= 2 && use_tensor && gemm_f16_tc_supported(m, w->n, w->k))
      return gemm_f16_tc((const half*)x, (const half*)w->w16, (const half*)w->bias, (half*)y, m, w->n, w->k,
                         (float*)workspace, (cudaStream_t)stream, true);
    return quic_gemm_f16(x, w->w16, w->bias, y, m, w->n, w->k, stream);
  }
  QUIC_REQUIRE(w->qw && w->sc && w->zp, QUIC_E_ARG, "w4a16_linear: null tensor");
  QUIC_REQUIRE(w->n > 0 && w->k > 0 && w->n % 32 == 0 && w->k % kGroup == 0, QUIC_E_SHAPE,
               "w4a16_linear: N must be a multiple of 32 and K of 128");
  QUIC_REQUIRE(m >= 0, QUIC_E_SHAPE, "w4a16_linear: negative M");
  if (m == 0) return QUIC_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (use_tensor && m >= kTensorMinRows && w->n % 128 == 0 && w->k % 64 == 0) {
    QUIC_REQUIRE(workspace != nullptr, QUIC_E_ARG, "w4a16_linear: tensor path needs a workspace");
    return w4a16_gemm_tc((const half*)x, *w, (half*)y, m, (float*)workspace, st, nullptr);
  }
  // the first 16 KB of the workspace belong to the tensor path's arrival counters
  float* part = workspace != nullptr ? static_cast<float*>(workspace) + 4096 : nullptr;
  const int ng = w->k / kGroup;
  int splits = (workspace != nullptr && m <= 8) ? gemv_splits(w->n, w->k) : 1;
  int gps = (ng + splits - 1) / splits;
  // keep the fp16 activation slice of 8 rows within ~64 KB of shared memory
  while (gps * kGroup * 2 * 8 > 65536) gps = (gps + 1) / 2;
  splits = (ng + gps - 1) / gps;
  QUIC_REQUIRE(splits == 1 || workspace != nullptr, QUIC_E_ARG,
               "w4a16_linear: K this large needs a workspace for split-K partials");
  const int nwarp = gps < 16 ? gps : 16;
  const int M = m == 1 ? 1 : 8;
  const int mchunks = (m + M - 1) / M;
  QUIC_REQUIRE(mchunks <= 65535, QUIC_E_SHAPE, "w4a16_linear: too many rows");
  const size_t smem = (size_t)M * gps * kGroup * 2 + (size_t)nwarp * M * 32 * 4;
  dim3 grid(w->n / 32, splits, mchunks);
  if (M == 1) {
    QUIC_CUDA(cudaFuncSetAttribute(w4_gemv_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)smem));
    w4_gemv_kernel<1><<<grid, nwarp * 32, smem, st>>>((const half*)x, *w, (half*)y, part, m, gps);
  } else {
    QUIC_CUDA(cudaFuncSetAttribute(w4_gemv_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)smem));
    w4_gemv_kernel<8><<<grid, nwarp * 32, smem, st>>>((const half*)x, *w, (half*)y, part, m, gps);
  }
  QUIC_CUDA(cudaGetLastError());
  if (splits > 1) {
    const size_t total = (size_t)m * w->n;
    splitk_finish_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        part, (const half*)w->bias, (half*)y, m, w->n, splits);
    QUIC_CUDA(cudaGetLastError());
  }
  return QUIC_OK;
}
