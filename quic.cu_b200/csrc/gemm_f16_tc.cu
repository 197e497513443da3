// Dense fp16 linear y[M, N] = x[M, K] . W[N, K]^T (+ bias) on tcgen05: the linears of the
// un-quantised model (the reference's second execution path, src/model.py:35-41 ->
// kernels/cuda/gemm.cu:36-82, cublasGemmEx with fp32 accumulation) for prefill and for decode
// steps of more than a few rows.
//
// Same "swap AB" mapping as the W4A16 GEMM and the tensor lm_head: 128 weight rows on the UMMA
// M side, MT activation rows on the N side, so a few batch rows do not waste a 128-row tile.
// Both operands are fp16 in global memory: both tiles arrive by TMA (no cluster multicast)
// already in the 128-byte swizzled layout, there are no dequantisation warps, and the main
// loop is: wait for a stage, issue four MMAs per 64-wide k block, release the stage.  The
// accumulator sits in tensor memory and is read back once with tcgen05.ld; the epilogue rounds
// to fp16 as the reference's GEMM output does and adds the bias in fp16.
//
// Roles: warps 0-3 epilogue (thread 0 issues the MMAs), warp 4 the TMA producer.  Every wait
// is bounded; a wait that runs out sets word 0 of the tensor path's error words and the CTA
// leaves with its tensor memory released.
#include "tc_common.cuh"

namespace quic {
namespace {

constexpr int kDenseStages = 4;
constexpr int kDenseThreads = 128 + 32;

template <int MT>
struct DenseSmem {
  static constexpr uint32_t kA = kTileN * 128;                              // 128 weight rows x 64 k
  static constexpr uint32_t kB = ((uint32_t)MT * 128u + 1023u) & ~1023u;    // MT activation rows x 64 k
  static constexpr uint32_t kStage = kA + kB;
  static constexpr uint32_t kTotal = kDenseStages * kStage + 1024;
};

struct DenseArgs {
  const half* bias;  // [N] or nullptr
  half* y;           // [M, N]
  float* part;       // split K: [splits][M][N] fp32 partial sums (then y and bias belong to the finish kernel)
  int m_total, n, k;
  int kb_per_split;  // 64-wide k blocks per CTA along grid.z
};

template <int MT>
__global__ void __launch_bounds__(kDenseThreads) gemm_f16_tc_kernel(const __grid_constant__ CUtensorMap tm_w,
                                                                    const __grid_constant__ CUtensorMap tm_x,
                                                                    const DenseArgs a, int* status) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kDenseStages];
  __shared__ __align__(8) uint64_t bar_empty[kDenseStages];
  __shared__ __align__(8) uint64_t bar_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int fail_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * kTileN;
  const int m0 = blockIdx.y * MT;
  const int kb0 = blockIdx.z * a.kb_per_split;
  const int nkb = min(a.k / kBlockK - kb0, a.kb_per_split);
  using L = DenseSmem<MT>;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr uint32_t kCols = MT < 32 ? 32 : MT;

  if (tid == 0) {
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
    for (int s = 0; s < kDenseStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_done), 1);
    fail_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_base_s)),
                 "r"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = tmem_base_s;
  const uint32_t idesc = umma_idesc_f16(MT);
  pdl_launch_dependents();

  if (warp == 4) {
    if (lane == 0) {
      // The weight tiles of the first ring pass do not depend on the previous kernel: they are
      // requested before the dependency wait, the activation tiles after it.  A stage's barrier
      // expects both.
      const int first = nkb < kDenseStages ? nkb : kDenseStages;
      for (int it = 0; it < first; ++it) {
        const uint32_t full = smem_u32(&bar_full[it]);
        mbar_expect_tx(full, L::kA + (uint32_t)MT * 128u);
        tma_load_2d(base + it * L::kStage, &tm_w, (kb0 + it) * kBlockK, n0, full);
      }
      pdl_wait();
      for (int it = 0; it < first; ++it)
        tma_load_2d(base + it * L::kStage + L::kA, &tm_x, (kb0 + it) * kBlockK, m0, smem_u32(&bar_full[it]));
      for (int it = first; it < nkb; ++it) {
        const int stage = it % kDenseStages;
        if (!mbar_wait(smem_u32(&bar_empty[stage]), ((it / kDenseStages) - 1) & 1)) {
          fail_s = 2;
          break;
        }
        const uint32_t a_s = base + stage * L::kStage, b_s = a_s + L::kA;
        const uint32_t full = smem_u32(&bar_full[stage]);
        mbar_expect_tx(full, L::kA + (uint32_t)MT * 128u);
        tma_load_2d(a_s, &tm_w, (kb0 + it) * kBlockK, n0, full);
        tma_load_2d(b_s, &tm_x, (kb0 + it) * kBlockK, m0, full);
      }
    }
  } else if (tid == 0) {
    for (int it = 0; it < nkb; ++it) {
      const int stage = it % kDenseStages;
      if (!mbar_wait(smem_u32(&bar_full[stage]), (it / kDenseStages) & 1)) {
        fail_s = 1;
        break;
      }
      tc_fence_after();
      const uint32_t a_s = base + stage * L::kStage, b_s = a_s + L::kA;
#pragma unroll
      for (int k = 0; k < kBlockK / 16; ++k)
        umma_f16(tmem_d, umma_desc_sw128(a_s + k * 32), umma_desc_sw128(b_s + k * 32), idesc,
                 (it > 0 || k > 0) ? 1u : 0u);
      if (it + kDenseStages < nkb) umma_commit(smem_u32(&bar_empty[stage]));
      if (it == nkb - 1) umma_commit(smem_u32(&bar_done));
    }
  }
  __syncwarp();

  if (warp < 4) {
    pdl_wait();  // y may still be read by an earlier kernel of the chain
    bool ok = mbar_wait_relaxed(smem_u32(&bar_done), 0, 32) && !fail_s;
    ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below is warp-collective
    tc_fence_after();
    if (!ok && tid == 0) atomicCAS(status, 0, ((fail_s ? fail_s : 3) << 16) | 0x4000 | ((int)blockIdx.x & 0x3fff));
    const int col = n0 + warp * 32 + lane;  // TMEM lane = weight row = output column
    const float bias = a.bias != nullptr ? __half2float(a.bias[col]) : 0.f;
    if (ok) {
#pragma unroll 1
      for (int c0 = 0; c0 < MT; c0 += 8) {
        if (m0 + c0 >= a.m_total) break;
        uint32_t r[8];
        const uint32_t taddr = tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                       "=r"(r[7])
                     : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int m = m0 + c0 + j;
          if (m >= a.m_total) continue;
          if (a.part != nullptr) {
            a.part[((size_t)blockIdx.z * a.m_total + m) * a.n + col] = __uint_as_float(r[j]);
            continue;
          }
          float o = __half2float(__float2half_rn(__uint_as_float(r[j])));
          if (a.bias != nullptr) o += bias;
          a.y[(size_t)m * a.n + col] = __float2half_rn(o);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(kCols) : "memory");
}

// y = fp16(sum of the split-K partials, in split order) (+ bias): four consecutive outputs per thread.
__global__ void gemm_f16_finish_kernel(const float* __restrict__ part, const half* __restrict__ bias,
                                       half* __restrict__ y, int m_total, int n, int splits) {
  const size_t idx = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const size_t total = (size_t)m_total * n;
  pdl_launch_dependents();
  pdl_wait();
  if (idx >= total) return;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < splits; ++s) {
    const float4 p = __ldcg(reinterpret_cast<const float4*>(part + (size_t)s * total + idx));
    v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
  }
  float o[4] = {v.x, v.y, v.z, v.w};
  const int col = (int)(idx % (size_t)n);
  half h[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float f = __half2float(__float2half_rn(o[j]));
    if (bias != nullptr) f += __half2float(bias[col + j]);
    h[j] = __float2half_rn(f);
  }
  *reinterpret_cast<uint2*>(y + idx) = *reinterpret_cast<const uint2*>(h);
}

// K splits for a problem whose tiles would leave most SMs idle: at most 16, at least two k
// blocks each, while the CTAs at most fill the SMs once.
int dense_splits(int m, int n, int k, int mt) {
  const int ctas = (n / kTileN) * ((m + mt - 1) / mt);
  const int nkb = k / kBlockK;
  int splits = 1;
  while (splits < 16 && ctas * splits * 2 <= 148 && nkb / (splits * 2) >= 2) splits *= 2;
  return splits;
}
int dense_mt(int m) { return m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128; }

template <int MT>
int run(const half* x, const half* w, const DenseArgs& a, int splits, cudaStream_t st, bool pdl) {
  CUtensorMap tm_w, tm_x;
  int rc = make_map(&tm_w, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, w, (uint64_t)a.n, (uint64_t)a.k, kTileN, kBlockK,
                    CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != QUIC_OK) return rc;
  rc = make_map(&tm_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x, (uint64_t)a.m_total, (uint64_t)a.k, MT, kBlockK,
                CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != QUIC_OK) return rc;
  int* status = tc_status_words();
  QUIC_REQUIRE(status != nullptr, QUIC_E_CUDA, "gemm_f16: no address for the tensor path's error words");
  const size_t smem = DenseSmem<MT>::kTotal;
  QUIC_CUDA(cudaFuncSetAttribute(gemm_f16_tc_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(a.n / kTileN, (a.m_total + MT - 1) / MT, splits);
  QUIC_CUDA(launch(gemm_f16_tc_kernel<MT>, grid, dim3(kDenseThreads), smem, st, pdl, tm_w, tm_x, a, status));
  return QUIC_OK;
}

}  // namespace

bool gemm_f16_tc_supported(int m, int n, int k) {
  return m >= 1 && n >= kTileN && n % kTileN == 0 && k >= kBlockK && k % kBlockK == 0 && (m + 127) / 128 <= 65535;
}

// Bytes of split-K workspace gemm_f16_tc may use for this shape (0: it never splits it).
int64_t gemm_f16_tc_workspace(int m, int n, int k) {
  if (!gemm_f16_tc_supported(m, n, k)) return 0;
  const int splits = dense_splits(m, n, k, dense_mt(m));
  return splits > 1 ? (int64_t)splits * m * n * 4 : 0;
}

// x fp16 [m, k] (row-major, 16-byte aligned), w fp16 [n, k], bias fp16 [n] or nullptr -> y fp16 [m, n].
// `ws` (gemm_f16_tc_workspace bytes, may be null): lets small problems split K over more CTAs.
int gemm_f16_tc(const half* x, const half* w, const half* bias, half* y, int m, int n, int k, float* ws,
                cudaStream_t st, bool pdl) {
  QUIC_REQUIRE(gemm_f16_tc_supported(m, n, k), QUIC_E_SHAPE,
               "gemm_f16: the tensor path needs N a multiple of 128 and K a multiple of 64");
  QUIC_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), QUIC_E_ARG,
               "gemm_f16: x and w must be 16-byte aligned");
  const int mt = dense_mt(m);
  int splits = ws != nullptr ? dense_splits(m, n, k, mt) : 1;
  const int nkb = k / kBlockK;
  DenseArgs a = {};
  a.bias = bias;
  a.y = y;
  a.m_total = m;
  a.n = n;
  a.k = k;
  a.kb_per_split = (nkb + splits - 1) / splits;
  splits = (nkb + a.kb_per_split - 1) / a.kb_per_split;
  a.part = splits > 1 ? ws : nullptr;
  int rc;
  switch (mt) {
    case 16: rc = run<16>(x, w, a, splits, st, pdl); break;
    case 32: rc = run<32>(x, w, a, splits, st, pdl); break;
    case 64: rc = run<64>(x, w, a, splits, st, pdl); break;
    default: rc = run<128>(x, w, a, splits, st, pdl); break;
  }
  if (rc != QUIC_OK || splits == 1) return rc;
  const size_t total = (size_t)m * n;
  QUIC_CUDA(launch(gemm_f16_finish_kernel, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0, st, true,
                   (const float*)ws, bias, y, m, n, splits));
  return QUIC_OK;
}

}  // namespace quic
