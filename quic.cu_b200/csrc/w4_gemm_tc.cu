// W4A16 GEMM for batch >= 16 on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   y[m, n] = sum_k x[m, k] * dequant(W)[n, k] (+ bias[n])      fp16 in/out, fp32 accumulate
//
// Replaces the reference's Marlin kernel (kernels/cuda/marlin.cu:1527, reached through
// src/quant/marlin.py:190) at the batch sizes where it tiles mma.sync; nothing of its
// structure is kept.  Mapping ("swap AB"): the 128 weight rows of a CTA tile sit on the
// M side of the UMMA (TMEM lanes), the batch rows on its N side (TMEM columns), so the
// accumulator of a 128 x MT tile is MT fp32 columns of tensor memory and a thread of the
// epilogue owns one output column n.
//
// Per 64-wide k block a CTA
//   1. loads 8 packed int32 words per weight row (thread t <-> row t, coalesced over rows),
//      dequantises them in registers exactly like the GEMV path ((q - zp) * s rounded once
//      to fp16) and writes the row's 128 bytes into the A stage in the K-major 128-byte
//      swizzled layout the UMMA shared-memory descriptor expects;
//   2. copies the x tile (MT rows x 128 bytes) into the B stage in the same layout;
//   3. makes the writes visible to the async proxy, and one thread issues four
//      tcgen05.mma (K = 16 each) that accumulate into TMEM, then commits them to the
//      stage's mbarrier so the stage can be refilled once the tensor core has read it.
// Three stages keep global loads, dequantisation and MMA overlapped.  Split-K CTAs write
// fp32 partials that a small kernel sums.  Every mbarrier wait is bounded: on a timeout
// the kernel records an error code, still frees its tensor memory and returns.
#include "decode_kernels.cuh"

namespace quic {
namespace {

constexpr int kTileN = 128;   // weight rows per CTA (UMMA M)
constexpr int kBlockK = 64;   // k per stage: 64 fp16 = one 128-byte swizzle row
constexpr int kStages = 3;
constexpr int kThreads = 128;
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ int g_tc_status;  // 0 = ok; otherwise (code << 16) | block of the first failure

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
// Bounded wait for the phase with the given parity; false on timeout.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);  // start address
  d |= (uint64_t)1 << 16;                    // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                    // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
  return d;
}
// kind::f16, fp16 x fp16 -> fp32, both operands K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc_f16(int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// Byte offset of 16-byte chunk c (0..7) of row r inside a swizzled tile.
__device__ __forceinline__ uint32_t sw128_offset(int r, int c) { return r * 128 + ((c ^ (r & 7)) << 4); }

struct GemmArgs {
  const half* x;  // [m_total, K]
  quic_w4_t w;
  half* y;         // [m_total, N]    (splits == 1)
  float* part;     // [splits, m_total, N] fp32 (splits > 1)
  int m_total;
  int kblocks_per_split;
};

template <int MT>  // batch rows per CTA tile (UMMA N): 16, 32, 64, 128 or 256
__global__ void __launch_bounds__(kThreads) w4a16_gemm_tc_kernel(const GemmArgs a) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bar_free[kStages];
  __shared__ __align__(8) uint64_t bar_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int fail_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * kTileN;
  const int split = blockIdx.y;
  const int m0 = blockIdx.z * MT;
  const int K = a.w.k, N = a.w.n;
  const int kb_total = K / kBlockK;
  const int kb0 = split * a.kblocks_per_split;
  const int kb1 = min(kb_total, kb0 + a.kblocks_per_split);

  // 1024-byte aligned stage buffers: A (16 KB) then B (MT * 128 bytes) per stage
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr uint32_t kABytes = kTileN * 128, kBBytes = MT * 128;
  constexpr uint32_t kStageBytes = kABytes + ((kBBytes + 1023u) & ~1023u);
  unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));

  constexpr uint32_t kCols = MT < 32 ? 32 : MT;  // power of two >= 32
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(smem_u32(&bar_free[s]), 1);
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

  const half* scp = reinterpret_cast<const half*>(a.w.sc);
  const int n = n0 + tid;  // this thread's weight row
  int it = 0;
  for (int kb = kb0; kb < kb1; ++kb, ++it) {
    const int stage = it % kStages;
    const uint32_t a_s = base + stage * kStageBytes, b_s = a_s + kABytes;
    unsigned char* a_g = gen_base + stage * kStageBytes;
    unsigned char* b_g = a_g + kABytes;

    // global loads first (they do not touch the stage)
    uint32_t q[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) q[j] = ldg_nc_u32(a.w.qw + ((size_t)kb * 8 + j) * N + n);
    const int g = (kb * kBlockK) / kGroup;
    const half2 s2 = __half2half2(scp[(size_t)g * N + n]);
    const half2 zp = zp_to_half2((a.w.zp[(size_t)g * (N >> 1) + (n >> 1)] >> (4 * (n & 1))) & 15);
    constexpr int kXChunks = MT * 8;  // 16-byte chunks of the x tile
    uint4 xv[(kXChunks + kThreads - 1) / kThreads];
#pragma unroll
    for (int i = 0; i < (kXChunks + kThreads - 1) / kThreads; ++i) {
      const int idx = tid + i * kThreads;
      const int r = idx >> 3, c = idx & 7;
      xv[i] = make_uint4(0, 0, 0, 0);
      if (idx < kXChunks && m0 + r < a.m_total)
        xv[i] = *reinterpret_cast<const uint4*>(a.x + (size_t)(m0 + r) * K + kb * kBlockK + 8 * c);
    }

    // the tensor core must have finished reading this stage (MMAs of iteration it - kStages)
    if (it >= kStages) {
      const uint32_t parity = ((it / kStages) - 1) & 1;
      if (!mbar_wait(smem_u32(&bar_free[stage]), parity)) fail_s = 1;
    }

    // dequantise and store the A row (natural k order inside each 16-byte chunk)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      half2 d[4];
      dequant8(q[j], zp, s2, d);  // d[p] = (k = p, k = p + 4)
      const uint32_t u0 = *reinterpret_cast<uint32_t*>(&d[0]), u1 = *reinterpret_cast<uint32_t*>(&d[1]);
      const uint32_t u2 = *reinterpret_cast<uint32_t*>(&d[2]), u3 = *reinterpret_cast<uint32_t*>(&d[3]);
      uint4 o;
      o.x = __byte_perm(u0, u1, 0x5410);  // (k0, k1)
      o.y = __byte_perm(u2, u3, 0x5410);  // (k2, k3)
      o.z = __byte_perm(u0, u1, 0x7632);  // (k4, k5)
      o.w = __byte_perm(u2, u3, 0x7632);  // (k6, k7)
      *reinterpret_cast<uint4*>(a_g + sw128_offset(tid, j)) = o;
    }
#pragma unroll
    for (int i = 0; i < (kXChunks + kThreads - 1) / kThreads; ++i) {
      const int idx = tid + i * kThreads;
      if (idx < kXChunks) *reinterpret_cast<uint4*>(b_g + sw128_offset(idx >> 3, idx & 7)) = xv[i];
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && !fail_s) {
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < kBlockK / 16; ++k)
        umma_f16(tmem_d, umma_desc_sw128(a_s + k * 32), umma_desc_sw128(b_s + k * 32), idesc,
                 (it > 0 || k > 0) ? 1u : 0u);
      umma_commit(smem_u32(&bar_free[stage]));
      if (kb == kb1 - 1) umma_commit(smem_u32(&bar_done));
    }
  }

  // wait for the whole accumulation, then read the accumulator out of tensor memory
  bool ok = !fail_s;
  if (ok && it > 0) ok = mbar_wait(smem_u32(&bar_done), 0);
  tc_fence_after();
  if (!ok && tid == 0) atomicCAS(&g_tc_status, 0, (1 << 16) | (int)blockIdx.x);

  if (ok && it > 0) {
    const int col = n0 + warp * 32 + lane;  // TMEM lane = tile row; warp w reads lanes 32w..32w+31
    const float bias =
        (a.w.bias != nullptr && gridDim.y == 1) ? __half2float(reinterpret_cast<const half*>(a.w.bias)[col]) : 0.f;
#pragma unroll 1
    for (int c0 = 0; c0 < MT; c0 += 8) {
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
        const float v = __uint_as_float(r[j]);
        if (gridDim.y == 1) {
          float o = __half2float(__float2half_rn(v));
          if (a.w.bias != nullptr) o += bias;
          a.y[(size_t)m * N + col] = __float2half_rn(o);
        } else {
          a.part[((size_t)split * a.m_total + m) * N + col] = v;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(kCols) : "memory");
}

__global__ void tc_splitk_finish_kernel(const float* __restrict__ part, const half* __restrict__ bias,
                                        half* __restrict__ y, int m_total, int N, int splits) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)m_total * N) return;
  float v = 0.f;
  for (int s = 0; s < splits; ++s) v += part[(size_t)s * m_total * N + idx];
  v = __half2float(__float2half_rn(v));
  if (bias) v += __half2float(bias[idx % N]);
  y[idx] = __float2half_rn(v);
}

template <int MT>
int run(const GemmArgs& a, int splits, cudaStream_t st) {
  constexpr uint32_t kABytes = kTileN * 128, kBBytes = MT * 128;
  constexpr uint32_t kStageBytes = kABytes + ((kBBytes + 1023u) & ~1023u);
  const size_t smem = (size_t)kStages * kStageBytes + 1024;
  QUIC_CUDA(cudaFuncSetAttribute(w4a16_gemm_tc_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem));
  dim3 grid(a.w.n / kTileN, splits, (a.m_total + MT - 1) / MT);
  w4a16_gemm_tc_kernel<MT><<<grid, kThreads, smem, st>>>(a);
  QUIC_CUDA(cudaGetLastError());
  return QUIC_OK;
}

}  // namespace

static void tc_plan(int m, int n, int k, int* mt_out, int* splits_out, int* per_out) {
  const int kb_total = k / kBlockK;
  const int tiles = n / kTileN;
  const int mt = m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128;
  const int mtiles = (m + mt - 1) / mt;
  // split K until roughly every SM has a CTA, at most 8 ways and at least 2 k blocks per CTA
  int splits = 1;
  while (splits < 8 && tiles * mtiles * splits * 2 <= 148 && kb_total / (splits * 2) >= 2) splits *= 2;
  const int per = (kb_total + splits - 1) / splits;
  *mt_out = mt;
  *per_out = per;
  *splits_out = (kb_total + per - 1) / per;
}

int64_t w4a16_gemm_tc_workspace(int m, int n, int k) {
  int mt, splits, per;
  tc_plan(m, n, k, &mt, &splits, &per);
  return splits > 1 ? (int64_t)splits * m * n * 4 : 0;
}

int w4a16_gemm_tc(const half* x, const quic_w4_t& w, half* y, int m, float* workspace, cudaStream_t st) {
  QUIC_REQUIRE(w.n % kTileN == 0 && w.k % kBlockK == 0, QUIC_E_SHAPE,
               "w4a16_linear: the tensor path needs N multiple of 128 and K multiple of 64");
  QUIC_REQUIRE(((uintptr_t)x % 16 == 0) && w.k % 8 == 0, QUIC_E_ARG, "w4a16_linear: x must be 16-byte aligned");
  int mt, splits, per;
  tc_plan(m, w.n, w.k, &mt, &splits, &per);
  QUIC_REQUIRE(splits == 1 || workspace != nullptr, QUIC_E_ARG, "w4a16_linear: split-K needs a workspace");
  GemmArgs a = {};
  a.x = x;
  a.w = w;
  a.y = y;
  a.part = workspace;
  a.m_total = m;
  a.kblocks_per_split = per;
  int rc;
  switch (mt) {
    case 16: rc = run<16>(a, splits, st); break;
    case 32: rc = run<32>(a, splits, st); break;
    case 64: rc = run<64>(a, splits, st); break;
    default: rc = run<128>(a, splits, st); break;
  }
  if (rc != QUIC_OK) return rc;
  if (splits > 1) {
    const size_t total = (size_t)m * w.n;
    tc_splitk_finish_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        workspace, (const half*)w.bias, y, m, w.n, splits);
    QUIC_CUDA(cudaGetLastError());
  }
  return QUIC_OK;
}

}  // namespace quic

// Error word of the tensor path: 0, or (code << 16 | block) of the first bounded wait that
// gave up since the last call.  Synchronises the device; meant for tests and debugging.
extern "C" int quic_w4a16_tensor_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, quic::g_tc_status, sizeof(int)) != cudaSuccess) return -1;
  int zero = 0;
  cudaMemcpyToSymbol(quic::g_tc_status, &zero, sizeof(int));
  return v;
}
