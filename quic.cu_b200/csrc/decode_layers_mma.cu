// The four W4A16 linears of a decoder layer for 2..16 batch rows: the fused structure of the
// one-row GEMV chain (decode_layers.cu) with the batch rows on the M side of
// mma.sync.m16n8k16, so the cost of a launch does not grow with the row count.
//
// Common shape: a CTA owns 32 output columns, warp g owns quantisation group g of the K range
// the CTA covers.  Lane (gid = lane / 4, tig = lane % 4) owns, for each of the warp's four
// 8-column n-tiles, column 8 nt + gid and the packed words 4 t + tig (t = 0..3) of the group:
// the same 16 words per lane as the one-row kernels read, dequantised BEFORE
// griddepcontrol.wait into the B fragments of the group's eight k16 steps (64 registers).  The
// k index of the mma is mapped to weights so that word 4 t + tig supplies steps 2 t and
// 2 t + 1 (pairs (i, i + 4) of the word, as dequant8 produces them); the activations sit in
// shared memory in the matching "perm8" order, so one 16-byte load is a row's A fragments of
// two steps.  After the wait: rows -> shared memory (norm / copy), 32 mma per warp, groups
// summed through shared memory, epilogue.
//
// What changed against the one-row chain besides the mma: every kernel writes a FINISHED
// fp16 tensor, so no consumer has to sum partial planes whose size grows with the row count:
//   * gate|up: a CTA owns 16 gate columns and the 16 up columns of the same index (all seven
//     groups), applies SwiGLU itself and writes the activation; 304 small CTAs, two or three
//     resident per SM;
//   * down: the five K splits of a column tile form a thread-block cluster; the partial sums
//     meet in the first CTA's shared memory (distributed shared memory), which adds the
//     residual and writes the new residual stream;
//   * attention merges its splits itself (last CTA to arrive), as in the large-batch step.
//
// Reference for the arithmetic of each piece: see decode_layers.cu (same rounding points).
#include "attn_warp.cuh"
#include "decode_kernels.cuh"

namespace quic {
namespace {

constexpr int kRows = 16;                 // batch rows a CTA handles (rows >= batch are zero)
constexpr int kXsStride = kHidden + 8;    // halves; 16 bytes of padding: the 8 rows of an A fragment load hit 8 bank groups
constexpr int kDownSpan = 8 * kGroup;     // k range of a down split (up to 8 groups)
constexpr int kXdStride = kDownSpan + 8;

struct BTile {
  uint32_t q[4][4];  // [n-tile][t]: packed word 4 t + tig of the lane's column
  half2 s2[4];       // scale of the column, both halves
  half2 zp[4];       // zero point in the form dequant8 takes
};

__device__ __forceinline__ uint32_t h2u(half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

// Weights of (columns n0 .. n0+31, group g) as the lane's packed words; they become B fragments
// on the fly (btile_mma), so that only 24 registers stay occupied across the dependency wait.
// `col_of(nt)` gives the first column of n-tile nt (the gate|up kernel mixes two column ranges).
template <typename ColFn>
__device__ __forceinline__ void load_btile(BTile& f, const quic_w4_t& w, int g, ColFn col_of, int gid, int tig) {
  half s[4];
  uint8_t zb[4];
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    const int col = col_of(nt) + gid;
    const int32_t* p = w.qw + ((size_t)g * kWordsPerGroup + tig) * w.n + col;
#pragma unroll
    for (int t = 0; t < 4; ++t) f.q[nt][t] = ldg_nc_u32(p + (size_t)(4 * t) * w.n);
    s[nt] = reinterpret_cast<const half*>(w.sc)[(size_t)g * w.n + col];
    zb[nt] = w.zp[(size_t)g * (w.n >> 1) + (col >> 1)];
  }
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    const int col = col_of(nt) + gid;
    f.s2[nt] = __half2half2(s[nt]);
    f.zp[nt] = zp_to_half2((zb[nt] >> (4 * (col & 1))) & 15);
  }
}

// acc[nt] += x(rows 0..15, the group's 128 k) . W(n-tile nt): xs points at the group's first
// k of row 0 (perm8 order), rows `stride` halves apart.  Word 4 t + tig supplies k16 steps 2 t
// and 2 t + 1 (pairs (i, i + 4) of the word, as dequant8 produces them).
__device__ __forceinline__ void btile_mma(float (&acc)[4][4], const BTile& f, const half* xs, int stride, int nb,
                                          int gid, int tig) {
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    uint4 lo = make_uint4(0u, 0u, 0u, 0u), hi = make_uint4(0u, 0u, 0u, 0u);
    if (gid < nb) lo = *reinterpret_cast<const uint4*>(xs + (size_t)gid * stride + 8 * (4 * t + tig));
    if (gid + 8 < nb) hi = *reinterpret_cast<const uint4*>(xs + (size_t)(gid + 8) * stride + 8 * (4 * t + tig));
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      half2 h[4];
      dequant8(f.q[nt][t], f.zp[nt], f.s2[nt], h);
      mma16816(acc[nt], lo.x, hi.x, lo.y, hi.y, h2u(h[0]), h2u(h[1]));
      mma16816(acc[nt], lo.z, hi.z, lo.w, hi.w, h2u(h[2]), h2u(h[3]));
    }
  }
}

// acc -> red[warp][row][32 columns] (fp32); column of acc[nt][e] is 8 nt + 2 tig + (e & 1), row gid + 8 (e >> 1)
__device__ __forceinline__ void store_partials(float* red, const float (&acc)[4][4], int warp, int nb, int gid, int tig) {
  float* base = red + (size_t)warp * kRows * 32;
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    if (gid < nb) *reinterpret_cast<float2*>(base + gid * 32 + 8 * nt + 2 * tig) = make_float2(acc[nt][0], acc[nt][1]);
    if (gid + 8 < nb)
      *reinterpret_cast<float2*>(base + (gid + 8) * 32 + 8 * nt + 2 * tig) = make_float2(acc[nt][2], acc[nt][3]);
  }
}

// 8 consecutive halves (natural order) -> perm8 order (x0,x4,x1,x5,x2,x6,x3,x7)
__device__ __forceinline__ uint4 to_perm8(uint4 v) {
  uint4 o;
  o.x = __byte_perm(v.x, v.z, 0x5410);
  o.y = __byte_perm(v.x, v.z, 0x7632);
  o.z = __byte_perm(v.y, v.w, 0x5410);
  o.w = __byte_perm(v.y, v.w, 0x7632);
  return o;
}

constexpr int kSsqStride = 32;  // floats per row of a statistics buffer: one per 32-column tile (28 used)

// Rows of fp16 [.., ncols] -> xs (perm8 order) by the whole CTA, eight rows' worth of 16-byte
// pieces per pass (piece p = t + T i, i < 4, of a pass belongs to thread t of T; all four loads
// in flight together).  With `ln_s` (norm weights in shared memory) the rows are RMS-normalised
// on the way (fp32 statistics, fp16 result, as the reference's rmsnorm kernel).  The row's sum
// of squares comes
//   * from `ssq_part` ([row][kSsqStride], one partial per 32-column tile, written by the
//     kernel that produced the rows): warp w sums the partials of rows w, w + 7, ... while the
//     pieces are in flight, or,
//   * when ssq_part is null (rows gathered from the embedding table), from the pieces
//     themselves: they wait in registers while per-warp sums meet in `part` ([warp][row],
//     zeroed by the caller before its dependency wait).  This form needs T = 2 * ncols / 8, so
//     that a pass holds whole rows.
// Either way the partials are summed in a fixed order, so a row's statistics do not depend on
// the batch it is in.  `src_of(row)` returns the row's source pointer.  Ends with a CTA barrier.
template <typename SrcFn>
__device__ __forceinline__ void stage_rows(half* xs, int stride, SrcFn src_of, int ncols, int nb, const half* ln_s,
                                           float* part, const float* ssq_part, float eps, half* raw_out = nullptr) {
  const int nvec = ncols >> 3, pieces = nb * nvec, T = blockDim.x, t = threadIdx.x;
  const int nwarps = T >> 5, warp = t >> 5, lane = t & 31;
  const bool given = ln_s != nullptr && ssq_part != nullptr;
#pragma unroll 1
  for (int p0 = 0; p0 < pieces; p0 += 4 * T) {
    uint4 v[4];
    int row[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int p = p0 + t + T * i;
      v[i] = make_uint4(0u, 0u, 0u, 0u);
      row[i] = -1;
      if (p < pieces) {
        row[i] = p / nvec;
        v[i] = __ldcg(reinterpret_cast<const uint4*>(src_of(row[i])) + (p - row[i] * nvec));
      }
    }
    if (given && p0 == 0) {
      // part[row] = 1 / rms(row), from the producer's per-tile sums
      float q[3];
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        const int r = warp + nwarps * j;
        q[j] = (r < nb && lane < kHidden / 32) ? __ldcg(ssq_part + r * kSsqStride + lane) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        const int r = warp + nwarps * j;
        const float ssq = warp_sum(q[j]);
        if (lane == 0 && r < nb) part[r] = rsqrtf(ssq * (1.0f / kHidden) + eps);
      }
      __syncthreads();
    }
    if (ln_s != nullptr && !given) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float ss = 0.f;
        const half2* h = reinterpret_cast<const half2*>(&v[i]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __half22float2(h[e]);
          ss += f.x * f.x + f.y * f.y;
        }
        // a warp's pieces are consecutive, so they lie in at most two rows
        const int ra = __shfl_sync(0xffffffffu, row[i], 0), rb = __shfl_sync(0xffffffffu, row[i], 31);
        const float sa = warp_sum(row[i] == ra ? ss : 0.f);
        if (lane == 0 && ra >= 0) part[warp * kRows + ra] = sa;
        if (rb != ra) {
          const float sb = warp_sum(row[i] == rb ? ss : 0.f);
          if (lane == 0 && rb >= 0) part[warp * kRows + rb] = sb;
        }
      }
      __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (row[i] >= 0) {
        const int c = p0 + t + T * i - row[i] * nvec;
        if (raw_out != nullptr) reinterpret_cast<uint4*>(raw_out + (size_t)row[i] * ncols)[c] = v[i];
        uint4 o = v[i];
        if (ln_s != nullptr) {
          float r;
          if (given) {
            r = part[row[i]];
          } else {
            float ssq = 0.f;
            for (int w = 0; w < nwarps; ++w) ssq += part[w * kRows + row[i]];
            r = rsqrtf(ssq * (1.0f / kHidden) + eps);
          }
          const uint4 wv = *reinterpret_cast<const uint4*>(ln_s + 8 * c);
          const half2* h = reinterpret_cast<const half2*>(&v[i]);
          const half2* w2 = reinterpret_cast<const half2*>(&wv);
          uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(h[e]), wf = __half22float2(w2[e]);
            ou[e] = h2u(__floats2half2_rn(f.x * r * wf.x, f.y * r * wf.y));
          }
        }
        *reinterpret_cast<uint4*>(xs + (size_t)row[i] * stride + 8 * c) = to_perm8(o);
      }
    }
  }
  __syncthreads();
}

// New residual rows -> global, with the sum of squares of the CTA's 32 columns of every row
// (of the fp16 values written) -> ssq_part[row][tile] for the next RMSNorm.  `sum_of(row, pr)`
// returns the fp32 linear output for columns n0 + 2 pr, + 1 of the row.  Sixteen consecutive
// threads share a row, so the row sum is four shuffles.
template <typename SumFn>
__device__ __forceinline__ void residual_epilogue(SumFn sum_of, const half* xres_in, half* xres_out, float* ssq_part,
                                                  int n0, int tile, int nb) {
  const int T = blockDim.x;
  for (int e0 = 0; e0 < nb * 16; e0 += T) {  // warp-uniform trip count
    const int e = e0 + threadIdx.x;
    const int row = e >> 4, pr = e & 15;
    float ss = 0.f;
    if (row < nb) {
      const float2 v = sum_of(row, pr);
      const size_t idx = (size_t)row * kHidden + n0 + 2 * pr;
      const float2 r = __half22float2(*reinterpret_cast<const half2*>(xres_in + idx));
      // the linear's output is an fp16 tensor in the reference; so is the sum
      const half2 h = __floats2half2_rn(r.x + __half2float(__float2half_rn(v.x)), r.y + __half2float(__float2half_rn(v.y)));
      *reinterpret_cast<half2*>(xres_out + idx) = h;
      const float2 f = __half22float2(h);
      ss = f.x * f.x + f.y * f.y;
    }
    ss += __shfl_xor_sync(0xffffffffu, ss, 8);
    ss += __shfl_xor_sync(0xffffffffu, ss, 4);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    if (pr == 0 && row < nb) ssq_part[row * kSsqStride + tile] = ss;
  }
}

// Norm weights -> shared memory and zeroed partial sums of squares ([7 warps][16 rows]);
// touches nothing an earlier kernel of the chain writes, so it runs before the dependency wait.
__device__ __forceinline__ void stage_ln(half* ln_s, float* part, const half* ln) {
  const int t = threadIdx.x;
  if (t < kHidden / 8) reinterpret_cast<uint4*>(ln_s)[t] = ldg_nc_u128(reinterpret_cast<const uint4*>(ln) + t);
  if (t < 7 * kRows) part[t] = 0.f;
  __syncthreads();
}

// ---------------------------------------------------------------------------
// K1: RMSNorm -> QKV -> bias -> RoPE -> q buffer / KV append.  grid 36, block 224.
// ---------------------------------------------------------------------------
struct QkvMmaArgs {
  quic_w4_t w;
  const half* ln;
  const half* embed;    // first layer: rows are gathered from the table
  const half* x_in;     // [batch][896] residual stream
  const float* ssq_in;  // [batch][kSsqStride] its per-tile sums of squares (not used by the first layer)
  half* x_copy;         // first layer: the gathered rows are written here (the layer's residual input)
  RowState rs;
  float eps;
  int32_t first_layer, vocab;
  const half* cos_t;
  const half* sin_t;
  int32_t max_pos;
  half* qbuf;
  half* kcache;
  half* vcache;
  int32_t s_max;
};

__global__ void __launch_bounds__(224, 3) qkv_mma_kernel(const QkvMmaArgs a) {
  __shared__ __align__(16) half xs[kRows * kXsStride];
  __shared__ __align__(16) float red[7 * kRows * 32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
  const int n0 = blockIdx.x * 32;
  const int nb = a.rs.batch < kRows ? a.rs.batch : kRows;

  __shared__ __align__(16) half ln_s[kHidden];
  __shared__ float ssq_s[7 * kRows];
  pdl_trigger_early();
  BTile bt;
  load_btile(bt, a.w, warp, [&](int nt) { return n0 + 8 * nt; }, gid, tig);
  stage_ln(ln_s, ssq_s, a.ln);
  pdl_wait();

  stage_rows(xs, kXsStride,
             [&](int row) -> const half* {
               if (!a.first_layer) return a.x_in + (size_t)row * kHidden;
               int tk = __ldcg(a.rs.tok + a.rs.rows[row]);
               tk = tk < 0 ? 0 : (tk >= a.vocab ? a.vocab - 1 : tk);
               return a.embed + (size_t)tk * kHidden;
             },
             kHidden, nb, ln_s, ssq_s, a.first_layer ? nullptr : a.ssq_in, a.eps,
             (a.first_layer && blockIdx.x == 0) ? a.x_copy : nullptr);
  float acc[4][4] = {};
  btile_mma(acc, bt, xs + warp * kGroup, kXsStride, nb, gid, tig);
  pdl_trigger_late();
  store_partials(red, acc, warp, nb, gid, tig);
  __syncthreads();

  // epilogue: one (row, column pair) per thread-iteration; the pair is a RoPE pair
  const int head = n0 >> 6;  // 0..13 q, 14..15 k, 16..17 v (a 32-column tile never straddles heads)
  for (int e = tid; e < nb * 16; e += 224) {
    const int row = e >> 4, pr = e & 15;
    float v0 = 0.f, v1 = 0.f;
#pragma unroll
    for (int g = 0; g < 7; ++g) {
      const float2 p = *reinterpret_cast<const float2*>(red + ((size_t)g * kRows + row) * 32 + 2 * pr);
      v0 += p.x;
      v1 += p.y;
    }
    const int col = n0 + 2 * pr;
    const float2 bias = a.w.bias ? __half22float2(*reinterpret_cast<const half2*>(
                                       reinterpret_cast<const half*>(a.w.bias) + col))
                                 : make_float2(0.f, 0.f);
    // fp16 linear output with bias, as the reference's GEMM writes it
    v0 = __half2float(__float2half_rn(__half2float(__float2half_rn(v0)) + bias.x));
    v1 = __half2float(__float2half_rn(__half2float(__float2half_rn(v1)) + bias.y));
    const int slot = a.rs.rows[row];
    int p = __ldcg(a.rs.pos + slot);
    const int pj = (col & 63) >> 1;
    float lo = v0, hi = v1;
    if (head < kHeads + kKvHeads) {
      const int pc = p < a.max_pos ? (p < 0 ? 0 : p) : a.max_pos - 1;
      const float cs = __half2float(a.cos_t[(size_t)pc * 32 + pj]), sn = __half2float(a.sin_t[(size_t)pc * 32 + pj]);
      lo = v0 * cs - v1 * sn;
      hi = v0 * sn + v1 * cs;
    }
    const half lo16 = __float2half_rn(lo), hi16 = __float2half_rn(hi);
    if (head < kHeads) {
      half* q = a.qbuf + ((size_t)row * kHeads + head) * kHeadDim;
      q[pj] = lo16;
      q[pj + 32] = hi16;
    } else if (p >= 0 && p < a.s_max) {
      const int kvh = (head - kHeads) & 1;
      half* base = head < kHeads + kKvHeads ? a.kcache : a.vcache;
      half* dst = base + (((size_t)slot * kKvHeads + kvh) * a.s_max + p) * kHeadDim;
      dst[pj] = lo16;
      dst[pj + 32] = hi16;
    }
  }
}

// ---------------------------------------------------------------------------
// K3: o_proj -> residual add.  grid 28, block 224.
// ---------------------------------------------------------------------------
struct OProjMmaArgs {
  quic_w4_t w;
  const half* attn;     // [batch][896]
  const half* xres_in;  // [batch][896]
  half* xres_out;
  float* ssq_out;  // [batch][kSsqStride]: sums of squares of the rows written, per 32-column tile
  int32_t batch;
};

__global__ void __launch_bounds__(224, 3) oproj_mma_kernel(const OProjMmaArgs a) {
  __shared__ __align__(16) half xs[kRows * kXsStride];
  __shared__ __align__(16) float red[7 * kRows * 32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
  const int n0 = blockIdx.x * 32;
  const int nb = a.batch < kRows ? a.batch : kRows;

  pdl_trigger_early();
  BTile bt;
  load_btile(bt, a.w, warp, [&](int nt) { return n0 + 8 * nt; }, gid, tig);
  pdl_wait();

  stage_rows(xs, kXsStride, [&](int row) { return a.attn + (size_t)row * kHidden; }, kHidden, nb, nullptr, nullptr,
             nullptr, 0.f);
  float acc[4][4] = {};
  btile_mma(acc, bt, xs + warp * kGroup, kXsStride, nb, gid, tig);
  pdl_trigger_late();
  store_partials(red, acc, warp, nb, gid, tig);
  __syncthreads();

  residual_epilogue(
      [&](int row, int pr) {
        float2 v = make_float2(0.f, 0.f);
#pragma unroll
        for (int g = 0; g < 7; ++g) {
          const float2 p = *reinterpret_cast<const float2*>(red + ((size_t)g * kRows + row) * 32 + 2 * pr);
          v.x += p.x;
          v.y += p.y;
        }
        return v;
      },
      a.xres_in, a.xres_out, a.ssq_out, n0, blockIdx.x, nb);
}

// ---------------------------------------------------------------------------
// K4: RMSNorm -> gate & up -> SwiGLU.  grid 304 (16 gate + 16 up columns each), block 224.
// ---------------------------------------------------------------------------
struct GateUpMmaArgs {
  quic_w4_t w;  // n = 9728: gate rows then up rows
  const half* ln;
  const half* xres;  // [batch][896]
  const float* ssq_in;  // [batch][kSsqStride] its per-tile sums of squares
  half* act;         // [batch][4864]
  int32_t batch;
  float eps;
};

__global__ void __launch_bounds__(224, 3) gateup_mma_kernel(const GateUpMmaArgs a) {
  __shared__ __align__(16) half xs[kRows * kXsStride];
  __shared__ __align__(16) float red[7 * kRows * 32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
  __shared__ __align__(16) half ln_s[kHidden];
  __shared__ float ssq_s[7 * kRows];
  const int c0 = blockIdx.x * 16;  // gate columns c0..c0+15 and up columns kInter + c0..
  const int nb = a.batch < kRows ? a.batch : kRows;

  pdl_trigger_early();
  BTile bt;  // n-tiles 0,1: gate; 2,3: up
  load_btile(bt, a.w, warp, [&](int nt) { return (nt < 2 ? 0 : kInter) + c0 + 8 * (nt & 1); }, gid, tig);
  stage_ln(ln_s, ssq_s, a.ln);
  pdl_wait();

  stage_rows(xs, kXsStride, [&](int row) { return a.xres + (size_t)row * kHidden; }, kHidden, nb, ln_s, ssq_s,
             a.ssq_in, a.eps);
  float acc[4][4] = {};
  btile_mma(acc, bt, xs + warp * kGroup, kXsStride, nb, gid, tig);
  pdl_trigger_late();
  store_partials(red, acc, warp, nb, gid, tig);
  __syncthreads();

  for (int e = tid; e < nb * 8; e += 224) {
    const int row = e >> 3, pr = e & 7;  // column pair 2 pr, 2 pr + 1 of the 16
    float g0 = 0.f, g1 = 0.f, u0 = 0.f, u1 = 0.f;
#pragma unroll
    for (int g = 0; g < 7; ++g) {
      const float* base = red + ((size_t)g * kRows + row) * 32;
      const float2 pg = *reinterpret_cast<const float2*>(base + 2 * pr);
      const float2 pu = *reinterpret_cast<const float2*>(base + 16 + 2 * pr);
      g0 += pg.x;
      g1 += pg.y;
      u0 += pu.x;
      u1 += pu.y;
    }
    // gate and up are fp16 linear outputs in the reference; the SwiGLU output is fp16 too
    const float a0 = silu_mul(__half2float(__float2half_rn(g0)), __half2float(__float2half_rn(u0)));
    const float a1 = silu_mul(__half2float(__float2half_rn(g1)), __half2float(__float2half_rn(u1)));
    *reinterpret_cast<half2*>(a.act + (size_t)row * kInter + c0 + 2 * pr) = __floats2half2_rn(a0, a1);
  }
}

// ---------------------------------------------------------------------------
// K5: down -> residual add.  grid (28, 5): CTA (tile, ks) covers the groups of K split ks
// (8, 8, 8, 7, 7) and writes its partial tile to plane ks of `partial`; the CTA of a tile that
// arrives last at the tile's counter sums the five planes in the order of ks (so the result
// does not depend on which CTA that is), adds the residual, writes the new residual stream and
// re-arms the counter.  No CTA waits for another.  block 256.
// ---------------------------------------------------------------------------
struct DownMmaArgs {
  quic_w4_t w;
  const half* act;      // [batch][4864]
  const half* xres_in;  // [batch][896]
  half* xres_out;
  float* ssq_out;       // [batch][kSsqStride]
  float* partial;       // [kDownSplits][batch][896] fp32
  int32_t* counters;    // [28], zero between launches
  int32_t batch;
};

__global__ void __launch_bounds__(256, 2) down_mma_kernel(const DownMmaArgs a) {
  __shared__ __align__(16) half xs[kRows * kXdStride];
  float* red = reinterpret_cast<float*>(xs);  // [8][16][32] fp32: reuses xs once every warp has read its fragments
  static_assert(8 * kRows * 32 * 4 <= kRows * kXdStride * 2, "partials fit the activation tile");
  __shared__ int last_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
  const int n0 = blockIdx.x * 32;
  const int ks = blockIdx.y;
  const int nb = a.batch < kRows ? a.batch : kRows;
  const int g0 = down_group_begin(ks), g1 = down_group_begin(ks + 1);
  const bool has = g0 + warp < g1;

  pdl_trigger_early();
  BTile bt;
  if (has) load_btile(bt, a.w, g0 + warp, [&](int nt) { return n0 + 8 * nt; }, gid, tig);
  pdl_wait();

  const int kspan = (g1 - g0) * kGroup;
  stage_rows(xs, kXdStride, [&](int row) { return a.act + (size_t)row * kInter + g0 * kGroup; }, kspan, nb, nullptr,
             nullptr, nullptr, 0.f);
  float acc[4][4] = {};
  if (has) btile_mma(acc, bt, xs + warp * kGroup, kXdStride, nb, gid, tig);
  pdl_trigger_late();
  __syncthreads();  // xs becomes red
  if (has) store_partials(red, acc, warp, nb, gid, tig);
  __syncthreads();

  // this CTA's partial tile -> plane ks
  for (int e = tid; e < nb * 16; e += 256) {
    const int row = e >> 4, pr = e & 15;
    float2 v = make_float2(0.f, 0.f);
    for (int g = 0; g < g1 - g0; ++g) {
      const float2 p = *reinterpret_cast<const float2*>(red + ((size_t)g * kRows + row) * 32 + 2 * pr);
      v.x += p.x;
      v.y += p.y;
    }
    __stcg(reinterpret_cast<float2*>(a.partial + ((size_t)ks * a.batch + row) * kHidden + n0 + 2 * pr), v);
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) last_s = atomicAdd(a.counters + blockIdx.x, 1) == kDownSplits - 1;
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  residual_epilogue(
      [&](int row, int pr) {
        float2 p[kDownSplits];
#pragma unroll
        for (int s = 0; s < kDownSplits; ++s)
          p[s] = __ldcg(reinterpret_cast<const float2*>(a.partial + ((size_t)s * a.batch + row) * kHidden + n0 + 2 * pr));
        float2 v = make_float2(0.f, 0.f);
#pragma unroll
        for (int s = 0; s < kDownSplits; ++s) {
          v.x += p[s].x;
          v.y += p[s].y;
        }
        return v;
      },
      a.xres_in, a.xres_out, a.ssq_out, n0, blockIdx.x, nb);
  if (tid == 0) a.counters[blockIdx.x] = 0;
}

}  // namespace

// One decoder layer's four linears for 2..16 rows (the attention launch sits between the first
// two and is the caller's).  ssq_*: per-tile sums of squares of a residual stream
// ([batch][32] fp32), written by the kernel that writes the stream and read by the RMSNorm of
// the kernel that consumes it.
cudaError_t launch_qkv_mma(const quic_w4_t& w, const half* ln, const half* embed, const half* x_in,
                           const float* ssq_in, half* x_copy, const RowState& rs, float eps, bool first_layer,
                           int vocab, const half* cos_t, const half* sin_t, int max_pos, half* qbuf, half* kcache,
                           half* vcache, int s_max, cudaStream_t st, bool pdl) {
  QkvMmaArgs a = {};
  a.w = w;
  a.ln = ln;
  a.embed = embed;
  a.x_in = x_in;
  a.ssq_in = ssq_in;
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
  return launch(qkv_mma_kernel, dim3(kQkvN / 32), dim3(224), 0, st, pdl, a);
}

cudaError_t launch_oproj_mma(const quic_w4_t& w, const half* attn, const half* xres_in, half* xres_out, float* ssq_out,
                             int batch, cudaStream_t st) {
  OProjMmaArgs a = {};
  a.w = w;
  a.attn = attn;
  a.xres_in = xres_in;
  a.xres_out = xres_out;
  a.ssq_out = ssq_out;
  a.batch = batch;
  return launch(oproj_mma_kernel, dim3(kHidden / 32), dim3(224), 0, st, true, a);
}

cudaError_t launch_gateup_mma(const quic_w4_t& w, const half* ln, const half* xres, const float* ssq_in, half* act,
                              int batch, float eps, cudaStream_t st) {
  GateUpMmaArgs a = {};
  a.w = w;
  a.ln = ln;
  a.xres = xres;
  a.ssq_in = ssq_in;
  a.act = act;
  a.batch = batch;
  a.eps = eps;
  return launch(gateup_mma_kernel, dim3(kInter / 16), dim3(224), 0, st, true, a);
}

cudaError_t launch_down_mma(const quic_w4_t& w, const half* act, const half* xres_in, half* xres_out, float* ssq_out,
                            float* partial, int32_t* counters, int batch, cudaStream_t st) {
  DownMmaArgs a = {};
  a.w = w;
  a.act = act;
  a.xres_in = xres_in;
  a.xres_out = xres_out;
  a.ssq_out = ssq_out;
  a.partial = partial;
  a.counters = counters;
  a.batch = batch;
  return launch(down_mma_kernel, dim3(kHidden / 32, kDownSplits), dim3(256), 0, st, true, a);
}

}  // namespace quic
