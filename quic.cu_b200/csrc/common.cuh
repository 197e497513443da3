// Shared device helpers for the sm_100a decode kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/quic_b200.h"

namespace quic {

constexpr int kHidden = QUIC_HIDDEN;
constexpr int kHeads = QUIC_HEADS;
constexpr int kKvHeads = QUIC_KV_HEADS;
constexpr int kHeadDim = QUIC_HEAD_DIM;
constexpr int kInter = QUIC_INTER;
constexpr int kGroup = QUIC_GROUP;
constexpr int kQkvN = QUIC_QKV_N;
constexpr int kWordsPerGroup = kGroup / 8;  // 16 int32 words of 8 nibbles

// ---- error reporting (host) -------------------------------------------------
void set_error(const char* msg);
int fail(int code, const char* msg);
#define QUIC_REQUIRE(cond, code, msg) \
  do {                                \
    if (!(cond)) return ::quic::fail((code), (msg)); \
  } while (0)
#define QUIC_CUDA(expr)                                            \
  do {                                                             \
    cudaError_t e__ = (expr);                                      \
    if (e__ != cudaSuccess) return ::quic::fail(QUIC_E_CUDA, cudaGetErrorString(e__)); \
  } while (0)

// ---- programmatic dependent launch -----------------------------------------
// A kernel launched with the programmatic-serialisation attribute may start
// while its predecessor is still running.  Everything before pdl_wait() may
// only touch memory no earlier kernel writes (weights); pdl_wait() returns
// once the predecessor grid has completed and its writes are visible.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// Where a kernel lets its dependent start: at its top (the dependent's weight
// prefetch then overlaps this whole kernel and dependents cascade several
// kernels deep) or, with -DQUIC_PDL_LATE, after its main loop (one kernel deep).
__device__ __forceinline__ void pdl_trigger_early() {
#ifndef QUIC_PDL_LATE
  pdl_launch_dependents();
#endif
}
__device__ __forceinline__ void pdl_trigger_late() {
#ifdef QUIC_PDL_LATE
  pdl_launch_dependents();
#endif
}
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Process-wide switch (quic_set_pdl): when 0 every kernel is launched with plain
// stream ordering.  For A/B timing and debugging only.
bool pdl_enabled();

// Launch helper: `pdl` chains the kernel to the previous launch on the stream.
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl && pdl_enabled()) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- small device utilities -------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ uint32_t ldg_nc_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_nc_u128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

__device__ __forceinline__ half2 u32_as_half2(uint32_t u) {
  return *reinterpret_cast<half2*>(&u);
}

// Position inside an 8-wide k slab after the (i, i+4) pairing used by the
// unpack: value k=8j+i is stored at 8j + perm8(i).  Slot 2p holds i=p, slot
// 2p+1 holds i=p+4, so that pair p of dequant8() multiplies slots (2p, 2p+1).
__host__ __device__ __forceinline__ int perm8(int i) { return ((i & 3) << 1) | (i >> 2); }
__host__ __device__ __forceinline__ int perm_k(int k) { return (k & ~7) | perm8(k & 7); }

// Unpack one int32 word (nibble i = weight k=8j+i, reference
// src/quant/checkpoint.py:29-30) to four half2 of dequantised weights:
// out[p] = ((q_p - zp) * s, (q_{p+4} - zp) * s).  `zp1024` is (1024+zp) in both
// halves: 0x6400|q is the fp16 number 1024+q, so the subtraction is exact, and
// the product is rounded once to fp16 exactly as the reference's Marlin path
// (kernels/cuda/marlin.cu:2290-2293, 2311-2313) and its dequantised-weight
// oracle do.
__device__ __forceinline__ void dequant8(uint32_t w, half2 zp1024, half2 s2, half2 out[4]) {
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    uint32_t t = ((w >> (4 * p)) & 0x000f000fu) | 0x64006400u;
    out[p] = __hmul2(__hsub2(u32_as_half2(t), zp1024), s2);
  }
}

__device__ __forceinline__ half2 zp_to_half2(int zp) {
  uint32_t t = 0x64006400u | (uint32_t)zp | ((uint32_t)zp << 16);
  return u32_as_half2(t);
}

// acc += dot(dequant(word), xs[0..7]) with xs in perm8 order, fp32.
__device__ __forceinline__ float dot8(const half2 w[4], const float* __restrict__ xs, float acc) {
  const float4 a = *reinterpret_cast<const float4*>(xs);
  const float4 b = *reinterpret_cast<const float4*>(xs + 4);
  float2 f;
  f = __half22float2(w[0]);
  acc = fmaf(f.x, a.x, acc);
  acc = fmaf(f.y, a.y, acc);
  f = __half22float2(w[1]);
  acc = fmaf(f.x, a.z, acc);
  acc = fmaf(f.y, a.w, acc);
  f = __half22float2(w[2]);
  acc = fmaf(f.x, b.x, acc);
  acc = fmaf(f.y, b.y, acc);
  f = __half22float2(w[3]);
  acc = fmaf(f.x, b.z, acc);
  acc = fmaf(f.y, b.w, acc);
  return acc;
}

// acc + a*b with fp16 operands and an fp32 accumulator in ONE instruction (PTX
// mixed-precision fma, sm_100+): the product of two fp16 numbers is exact in
// fp32, so this equals convert-then-FFMA without the two conversions.
__device__ __forceinline__ float fma_h(float acc, half a, half b) {
  asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(acc) : "h"(__half_as_ushort(a)), "h"(__half_as_ushort(b)));
  return acc;
}

// acc[p] += dot of dequantised pair p with the matching activation pair; xs holds
// 8 fp16 activations of one k slab in perm8 order (one 16-byte shared load).
__device__ __forceinline__ void dot8_h(const half2 w[4], const half* __restrict__ xs, float acc[4]) {
  const uint4 xv = *reinterpret_cast<const uint4*>(xs);
  const half2* x2 = reinterpret_cast<const half2*>(&xv);
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    acc[p] = fma_h(acc[p], __low2half(w[p]), __low2half(x2[p]));
    acc[p] = fma_h(acc[p], __high2half(w[p]), __high2half(x2[p]));
  }
}

__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.0f + __expf(-g))) * u; }

}  // namespace quic
