// Tied fp16 lm_head of the tensor-core decode step (2..128 rows) on tcgen05, fused with the
// greedy argmax.
//
// Replaces cuBLAS lm_head + torch.argmax of the reference (src/model.py:301 ->
// kernels/cuda/gemm.cu:36, src/engine.py:104) when the GEMV kernel of lm_head.cu would have
// to re-read the 272 MB table once per 8 batch rows.  Same "swap AB" mapping as the W4A16
// GEMM: 128 vocabulary rows on the UMMA M side, the batch on the N side.  Both operands
// are fp16 in global memory, so both tiles arrive by TMA already in the 128-byte swizzled
// layout and the main loop is only: wait for a stage, issue four MMAs, release the stage.
// The epilogue rounds the logits to fp16 (the reference's logits are an fp16 tensor),
// optionally stores them, reduces (value, index) over the tile's 128 rows with ties going
// to the lower index (kernels/cuda/sampler.cu:38-40) and folds the tile's candidate of every
// batch row into one 64-bit atomic maximum per row; the CTA that arrives last at a counter
// decodes the maxima, publishes the tokens, advances the slot state and re-arms the maxima.
#include "tc_common.cuh"

namespace quic {
namespace {

constexpr int kLmStages = 3;  // 3 x 24 KB at 64 rows: three CTAs share an SM, so loads, MMAs and epilogues of different tiles overlap
constexpr int kLmThreads = 128 + 32;  // 4 epilogue warps (thread 0 issues MMAs) + 1 TMA warp

template <int MT>
struct LmSmem {
  static constexpr uint32_t kA = kTileN * 128;
  static constexpr uint32_t kB = ((uint32_t)MT * 128u + 1023u) & ~1023u;
  static constexpr uint32_t kStage = kA + kB;
  static constexpr uint32_t kTotal = kLmStages * kStage + 1024;
};

template <int MT>
__global__ void __launch_bounds__(kLmThreads) lm_head_tc_kernel(const __grid_constant__ CUtensorMap tm_e,
                                                                const __grid_constant__ CUtensorMap tm_x,
                                                                const LmHeadArgs a, int* status) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kLmStages];
  __shared__ __align__(8) uint64_t bar_empty[kLmStages];
  __shared__ __align__(8) uint64_t bar_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int fail_s;
  __shared__ int last_flag;
  __shared__ uint32_t cand_key[4][MT];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x, ntiles = gridDim.x;
  const int n0 = tile * kTileN;
  constexpr int nkb = kHidden / kBlockK;  // 14
  // Tiles start at different k blocks so that the CTAs running together do not all ask L2
  // for the same activation lines at the same moment.
  const int rot = tile % nkb;
  using L = LmSmem<MT>;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr uint32_t kCols = MT < 32 ? 32 : MT;

  if (tid == 0) {
    tma_prefetch_desc(&tm_e);
    tma_prefetch_desc(&tm_x);
    for (int s = 0; s < kLmStages; ++s) {
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
  pdl_wait();  // the normalised activations come from the previous kernel

  if (warp == 4) {
    if (lane == 0) {
      for (int it = 0; it < nkb; ++it) {
        const int stage = it % kLmStages;
        if (it >= kLmStages && !mbar_wait(smem_u32(&bar_empty[stage]), ((it / kLmStages) - 1) & 1)) {
          fail_s = 2;
          break;
        }
        const uint32_t a_s = base + stage * L::kStage, b_s = a_s + L::kA;
        const uint32_t full = smem_u32(&bar_full[stage]);
        mbar_expect_tx(full, L::kA + (uint32_t)MT * 128u);
        const int kb = (it + rot) % nkb;
        tma_load_2d(a_s, &tm_e, kb * kBlockK, n0, full);
        tma_load_2d(b_s, &tm_x, kb * kBlockK, 0, full);
      }
    }
  } else if (tid == 0) {
    for (int it = 0; it < nkb; ++it) {
      const int stage = it % kLmStages;
      if (!mbar_wait(smem_u32(&bar_full[stage]), (it / kLmStages) & 1)) {
        fail_s = 1;
        break;
      }
      tc_fence_after();
      const uint32_t a_s = base + stage * L::kStage, b_s = a_s + L::kA;
#pragma unroll
      for (int k = 0; k < kBlockK / 16; ++k)
        umma_f16(tmem_d, umma_desc_sw128(a_s + k * 32), umma_desc_sw128(b_s + k * 32), idesc,
                 (it > 0 || k > 0) ? 1u : 0u);
      umma_commit(smem_u32(&bar_empty[stage]));
      if (it == nkb - 1) umma_commit(smem_u32(&bar_done));
    }
  }
  __syncwarp();

  if (warp < 4) {
    // every epilogue thread waits for the accumulation itself (bounded)
    bool ok = mbar_wait(smem_u32(&bar_done), 0) && !fail_s;
    ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below is warp-collective
    tc_fence_after();
    if (!ok && lane == 0 && warp == 0) atomicCAS(status, 0, ((fail_s ? fail_s : 3) << 16) | 0x8000 | (tile & 0x7fff));
    const int row = n0 + warp * 32 + lane;
#pragma unroll 1
    for (int c0 = 0; c0 < MT; c0 += 8) {
      uint32_t r[8];
      const uint32_t taddr = tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
      if (ok) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                       "=r"(r[7])
                     : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = 0xff800000u;  // -inf
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int m = c0 + j;
        const half h = __float2half_rn(__uint_as_float(r[j]));
        if (a.logits != nullptr && m < a.batch && ok) a.logits[(size_t)m * a.vocab + row] = h;
        // (fp16 logit, row) as one unsigned key whose order is "larger logit, then lower
        // row": the warp maximum is a single redux instruction.
        const uint32_t bits = __half_as_ushort(h);
        const uint32_t ordered = (bits & 0x8000u) ? (~bits & 0xffffu) : (bits | 0x8000u);
        const uint32_t nan_safe = ((bits & 0x7fffu) > 0x7c00u) ? 0u : ordered;  // NaN never wins
        const uint32_t key = (nan_safe << 16) | (uint32_t)(127 - (warp * 32 + lane));
        const uint32_t top = __reduce_max_sync(0xffffffffu, key);
        if (lane == 0) cand_key[warp][m] = top;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(kCols) : "memory");

  // Tile candidate per batch row -> one 64-bit atomic maximum per row.  The key orders by
  // "larger logit, then lower vocabulary index" (argmax_kernel's tie rule, sampler.cu:38-40);
  // zero means "no finite logit yet".
  for (int m = tid; m < MT && m < a.batch; m += kLmThreads) {
    uint32_t k = cand_key[0][m];
#pragma unroll
    for (int w = 1; w < 4; ++w) k = max(k, cand_key[w][m]);
    const uint32_t ordered = k >> 16;
    const uint32_t index = (uint32_t)n0 + 127u - (k & 0xffffu);
    if (ordered != 0u)
      atomicMax(a.keys + m, ((unsigned long long)ordered << 32) | (unsigned long long)(0xffffffffu - index));
  }

  // the CTA that arrives last turns the keys into tokens and re-arms them
  __threadfence();
  __syncthreads();
  if (tid == 0) last_flag = (atomicAdd(a.counter, 1) == ntiles - 1);
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  int step = 0;
  if (a.step_counter != nullptr) step = *a.step_counter;
  for (int b = tid; b < a.batch; b += kLmThreads) {
    const unsigned long long key = __ldcg(a.keys + b);
    a.keys[b] = 0ull;
    const int token = key == 0ull ? 0 : (int)(0xffffffffu - (uint32_t)(key & 0xffffffffull));
    if (a.argmax_out != nullptr) a.argmax_out[b] = token;
    if (a.rows != nullptr) {
      const int slot = a.rows[b];
      a.tok[slot] = token;
      a.pos[slot] = a.pos[slot] + 1;
      if (a.out_tokens != nullptr) a.out_tokens[(size_t)(step % a.ring) * a.n_slots + slot] = token;
    }
  }
  __syncthreads();
  if (tid == 0) {
    *a.counter = 0;
    __threadfence();  // the new positions and tokens are visible before the step counter moves
    if (a.step_counter != nullptr) *a.step_counter = step + 1;
  }
}

template <int MT>
int run(const LmHeadArgs& a, cudaStream_t st) {
  CUtensorMap tm_e, tm_x;
  int rc = make_map(&tm_e, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.embed, (uint64_t)a.vocab, kHidden, kTileN, kBlockK,
                    CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != QUIC_OK) return rc;
  rc = make_map(&tm_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.x_normed, (uint64_t)a.batch, kHidden, MT, kBlockK,
                CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != QUIC_OK) return rc;
  int* status = tc_status_words();  // word 1 is this kernel's
  QUIC_REQUIRE(status != nullptr, QUIC_E_CUDA, "lm_head: no address for the tensor path's error words");
  status += 1;
  const size_t smem = LmSmem<MT>::kTotal;
  QUIC_CUDA(cudaFuncSetAttribute(lm_head_tc_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  QUIC_CUDA(launch(lm_head_tc_kernel<MT>, dim3(a.vocab / kTileN), dim3(kLmThreads), smem, st, true, tm_e, tm_x, a,
                   status));
  return QUIC_OK;
}

}  // namespace

bool lm_head_tc_supported(int batch, int vocab) { return batch >= 2 && batch <= 128 && vocab % kTileN == 0; }
int lm_head_tc_tiles(int vocab) { return vocab / kTileN; }

// x_normed rows [batch, 896] -> logits / argmax; the best_* arrays hold batch x (vocab / 128) entries.
int launch_lm_head_tc(const LmHeadArgs& a, cudaStream_t st) {
  QUIC_REQUIRE(a.x_normed != nullptr && lm_head_tc_supported(a.batch, a.vocab), QUIC_E_SHAPE,
               "lm_head: the tensor path needs 2..128 normalised rows and a vocabulary multiple of 128");
  QUIC_REQUIRE(((uintptr_t)a.embed % 16 == 0) && ((uintptr_t)a.x_normed % 16 == 0), QUIC_E_ARG,
               "lm_head: tensors must be 16-byte aligned");
  if (a.batch <= 16) return run<16>(a, st);
  if (a.batch <= 32) return run<32>(a, st);
  if (a.batch <= 64) return run<64>(a, st);
  return run<128>(a, st);
}

}  // namespace quic

