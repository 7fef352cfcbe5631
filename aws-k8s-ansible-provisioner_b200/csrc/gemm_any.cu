// gemm_any.cu -- C = A . W^T for operands of ANY shape and either precision (bf16 or fp32 elements, fp32 accumulation
// by plain fused multiply-adds: no reduced-precision matrix mode), as one strided batch or as ragged groups.
//
// The tcgen05 projections (gemm_tc.cu and friends) are built for bf16 operands whose sizes are multiples of their tiles.
// Models with a layer list bring shapes that are not (a latent of 96, 10 experts of 80 rows, a vocabulary of 500), a
// true-fp32 mode, per-head products against a slice of a wider activation row, and experts that each see their own
// subset of the tokens.  This kernel takes all of them:
//   * strided batch: blockIdx.z picks (A + z * a_bs, W + z * w_bs, C + z * c_bs): one launch for all heads of an
//     absorbed-query or value up-projection;
//   * ragged groups (routed experts): a device-built list of row tiles, each belonging to one group; rows of a group are
//     slots [group_offsets[g], group_offsets[g + 1]) of a token permutation, A rows are gathered through a_rows (slot ->
//     row of A) and the group's weights start at W + g * w_bs;
//   * epilogues: store (fp32 or bf16), squared ReLU then store, or add into an fp32 C (the residual stream).
// Tile 64 x 64 x 16, 256 threads, 4 x 4 outputs per thread, operands staged in shared memory as fp32; every global
// access is bounds-checked, so no size needs padding.  Rows of one output are summed in k order by one thread: the
// result of a row does not depend on which other rows share its tile.
//
// bf16 operands take the tensor-core form of the same tile (gemm_any_mma_kernel: warp-level 16 x 16 x 16 bf16 MMAs with
// fp32 accumulators, four warps of 32 x 32 outputs, 64 x 32 operand slabs staged with 16-byte loads when rows are
// 16-byte aligned and element by element when they are not); the fp32 form stays on plain FMAs because a true-fp32
// product has no tensor-core mode.  Same grid, same epilogues, same independence of a row from its tile mates.
//
// Few rows (a decode step: M <= 64 per batch, or experts that see a handful of tokens each) take gemm_any_rows_kernel
// instead: the product is then a stream of weights, not arithmetic.  The rows are staged in shared memory once per CTA,
// every warp walks two weight rows at a time with 16-byte loads (eight in flight per lane) and keeps one accumulator per
// staged row; a CTA covers 8 to 64 weight rows (8 while that still leaves every SM several CTAs).
#include <mma.h>

#include "kernels.h"

namespace b2 {

namespace {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename T>
__device__ __forceinline__ float ldf(const T* p);
template <>
__device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) gemm_any_kernel(AnyGemm g) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  const TA* A = reinterpret_cast<const TA*>(g.A);
  const TW* W = reinterpret_cast<const TW*>(g.W);
  TC* C = reinterpret_cast<TC*>(g.C);
  int row0, row_end;  // slots (ragged) or rows (dense) of this tile
  if (g.tile_group != nullptr) {
    if ((int)blockIdx.x >= *g.n_tiles) return;
    const int grp = g.tile_group[blockIdx.x];
    row0 = g.tile_row0[blockIdx.x];
    row_end = min(row0 + BM, g.group_offsets[grp + 1]);
    W += (size_t)grp * g.w_bs;
  } else {
    row0 = blockIdx.x * BM;
    row_end = min(row0 + BM, g.M);
    A += (size_t)blockIdx.z * g.a_bs;
    W += (size_t)blockIdx.z * g.w_bs;
    C += (size_t)blockIdx.z * g.c_bs;
  }
  const int n0 = blockIdx.y * BN;
  // loader mapping: thread -> (row r of the tile, 4 consecutive k)
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  long a_row = -1;
  if (row0 + lr < row_end) a_row = g.a_rows ? (long)g.a_rows[row0 + lr] : (long)(row0 + lr);
  const long w_row = (n0 + lr < g.N) ? (long)(n0 + lr) : -1;
  const int tx = tid & 15, ty = tid >> 4;  // outputs: rows ty*4.., cols tx*4..
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < g.K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      As[lk + j][lr] = (a_row >= 0 && k < g.K) ? ldf(A + a_row * g.lda + k) : 0.f;
      Ws[lk + j][lr] = (w_row >= 0 && k < g.K) ? ldf(W + w_row * g.ldw + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 w = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + ty * 4 + i;
    if (r >= row_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= g.N) continue;
      float v = acc[i][j] * g.alpha;
      TC* dst = C + (size_t)r * g.ldc + n;
      if (g.epilogue == ANY_EPI_RELU2) {
        v = fmaxf(v, 0.f);
        v = v * v;
      }
      if (g.epilogue == ANY_EPI_ADD) {
        if constexpr (sizeof(TC) == 4) *dst = (TC)((float)*dst + v);
      } else {
        if constexpr (sizeof(TC) == 4) *dst = v;
        else *dst = __float2bfloat16_rn(v);
      }
    }
  }
}

constexpr int MK = 32, MLD = MK + 8;  // k-slab of the MMA form and its padded row stride in shared memory (elements)

template <typename TC>
__global__ void __launch_bounds__(128) gemm_any_mma_kernel(AnyGemm g) {
  using namespace nvcuda;
  __shared__ __align__(32) unsigned char smem_raw[BM * (BN + 4) * 4];  // operand slabs during the k loop, the fp32 tile afterwards
  bf16* As = reinterpret_cast<bf16*>(smem_raw);                         // [BM][MLD]
  bf16* Ws = As + BM * MLD;                                             // [BN][MLD]
  float* Cs = reinterpret_cast<float*>(smem_raw);                       // [BM][BN + 4]
  __shared__ long a_rows_s[BM];
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5;
  const bf16* A = reinterpret_cast<const bf16*>(g.A);
  const bf16* W = reinterpret_cast<const bf16*>(g.W);
  TC* C = reinterpret_cast<TC*>(g.C);
  int row0, row_end;
  if (g.tile_group != nullptr) {
    if ((int)blockIdx.x >= *g.n_tiles) return;
    const int grp = g.tile_group[blockIdx.x];
    row0 = g.tile_row0[blockIdx.x];
    row_end = min(row0 + BM, g.group_offsets[grp + 1]);
    W += (size_t)grp * g.w_bs;
  } else {
    row0 = blockIdx.x * BM;
    row_end = min(row0 + BM, g.M);
    A += (size_t)blockIdx.z * g.a_bs;
    W += (size_t)blockIdx.z * g.w_bs;
    C += (size_t)blockIdx.z * g.c_bs;
  }
  const int n0 = blockIdx.y * BN;
  if (tid < BM) a_rows_s[tid] = (row0 + tid < row_end) ? (g.a_rows ? (long)g.a_rows[row0 + tid] : (long)(row0 + tid)) : -1;
  __syncthreads();
  // 16-byte loads need every row start and every k offset on a 16-byte boundary
  const bool a_vec = (g.lda % 8 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0);
  const bool w_vec = (g.ldw % 8 == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0);
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[2][2];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) wmma::fill_fragment(acc[i][j], 0.f);
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
  for (int k0 = 0; k0 < g.K; k0 += MK) {
    // stage: 64 rows x 32 k of each operand = 256 chunks of 8 elements; two chunks per thread and operand
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int ch = tid + it * 128, r = ch >> 2, kc = (ch & 3) * 8, k = k0 + kc;
      uint4 va = make_uint4(0, 0, 0, 0), vw = make_uint4(0, 0, 0, 0);
      const long ar = a_rows_s[r];
      if (ar >= 0) {
        const bf16* src = A + ar * g.lda + k;
        if (a_vec && k + 8 <= g.K) va = *reinterpret_cast<const uint4*>(src);
        else {
          bf16* e = reinterpret_cast<bf16*>(&va);
          for (int j = 0; j < 8; ++j)
            if (k + j < g.K) e[j] = src[j];
        }
      }
      if (n0 + r < g.N) {
        const bf16* src = W + (long)(n0 + r) * g.ldw + k;
        if (w_vec && k + 8 <= g.K) vw = ld_stream(src);
        else {
          bf16* e = reinterpret_cast<bf16*>(&vw);
          for (int j = 0; j < 8; ++j)
            if (k + j < g.K) e[j] = src[j];
        }
      }
      *reinterpret_cast<uint4*>(As + r * MLD + kc) = va;
      *reinterpret_cast<uint4*>(Ws + r * MLD + kc) = vw;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MK; kk += 16) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> fa[2];
      wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> fb[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) wmma::load_matrix_sync(fa[i], As + (wm + 16 * i) * MLD + kk, MLD);
#pragma unroll
      for (int j = 0; j < 2; ++j) wmma::load_matrix_sync(fb[j], Ws + (wn + 16 * j) * MLD + kk, MLD);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) wmma::mma_sync(acc[i][j], fa[i], fb[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) wmma::store_matrix_sync(Cs + (wm + 16 * i) * (BN + 4) + wn + 16 * j, acc[i][j], BN + 4, wmma::mem_row_major);
  __syncthreads();
  for (int idx = tid; idx < BM * BN; idx += 128) {
    const int rr = idx / BN, cc = idx - rr * BN;
    const int r = row0 + rr, n = n0 + cc;
    if (r >= row_end || n >= g.N) continue;
    float v = Cs[rr * (BN + 4) + cc] * g.alpha;
    TC* dst = C + (size_t)r * g.ldc + n;
    if (g.epilogue == ANY_EPI_RELU2) {
      v = fmaxf(v, 0.f);
      v = v * v;
    }
    if (g.epilogue == ANY_EPI_ADD) {
      if constexpr (sizeof(TC) == 4) *dst = (TC)((float)*dst + v);
    } else {
      if constexpr (sizeof(TC) == 4) *dst = v;
      else *dst = __float2bfloat16_rn(v);
    }
  }
}

// ---- few rows: weight-streaming form ----
constexpr int RB = 16, ROWS_NPB = 8;   // staged rows per pass; fewest weight rows per CTA (4 warps x one pair)

template <typename T>
__device__ __forceinline__ void load8(const T* p, int k, int K, bool vec, float* f);
template <>
__device__ __forceinline__ void load8<bf16>(const bf16* p, int k, int K, bool vec, float* f) {
  if (vec && k + 8 <= K) {
    unpack8(*reinterpret_cast<const uint4*>(p + k), f);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = k + j < K ? __bfloat162float(p[k + j]) : 0.f;
  }
}
template <>
__device__ __forceinline__ void load8<float>(const float* p, int k, int K, bool vec, float* f) {
  if (vec && k + 8 <= K) {
    const float4 a = *reinterpret_cast<const float4*>(p + k), b = *reinterpret_cast<const float4*>(p + k + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = k + j < K ? p[k + j] : 0.f;
  }
}

// eight weights as they lie in memory (16 or 32 bytes), widened only when they are used: four k-steps of two weight rows stay in
// flight per lane without holding 64 floats
template <typename T>
struct Raw8;
template <>
struct Raw8<bf16> {
  uint4 v;
  __device__ __forceinline__ void load(const bf16* p, int k, int K, bool vec) {
    if (vec && k + 8 <= K) v = ld_stream(p + k);
    else {
      bf16* e = reinterpret_cast<bf16*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = k + j < K ? p[k + j] : __float2bfloat16_rn(0.f);
    }
  }
  __device__ __forceinline__ void widen(float* f) const { unpack8(v, f); }
};
template <>
struct Raw8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p, int k, int K, bool vec) {
    if (vec && k + 8 <= K) {
      a = *reinterpret_cast<const float4*>(p + k);
      b = *reinterpret_cast<const float4*>(p + k + 4);
    } else {
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = k + j < K ? p[k + j] : 0.f;
      a = make_float4(f[0], f[1], f[2], f[3]);
      b = make_float4(f[4], f[5], f[6], f[7]);
    }
  }
  __device__ __forceinline__ void widen(float* f) const {
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
};

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(128) gemm_any_rows_kernel(AnyGemm g, int rows_per_pass, int npb) {
  extern __shared__ __align__(16) unsigned char rows_smem[];   // [rows_per_pass][Kp] of TA, Kp = K rounded up to 8
  TA* As = reinterpret_cast<TA*>(rows_smem);
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const TA* A = reinterpret_cast<const TA*>(g.A);
  const TW* W = reinterpret_cast<const TW*>(g.W);
  TC* C = reinterpret_cast<TC*>(g.C);
  int row_lo, row_hi;
  if (g.group_offsets != nullptr) {   // ragged: blockIdx.y = group
    row_lo = g.group_offsets[blockIdx.y];
    row_hi = g.group_offsets[blockIdx.y + 1];
    if (row_lo >= row_hi) return;
    W += (size_t)blockIdx.y * g.w_bs;
  } else {
    row_lo = 0;
    row_hi = g.M;
    A += (size_t)blockIdx.z * g.a_bs;
    W += (size_t)blockIdx.z * g.w_bs;
    C += (size_t)blockIdx.z * g.c_bs;
  }
  const int K = g.K, Kp = (K + 7) & ~7;
  const bool a_vec = (g.lda % 8 == 0) && ((reinterpret_cast<uintptr_t>(A) & 31) == 0);
  const bool w_vec = (g.ldw % 8 == 0) && ((reinterpret_cast<uintptr_t>(W) & 31) == 0);
  const int n_base = blockIdx.x * npb;
  for (int r0 = row_lo; r0 < row_hi; r0 += rows_per_pass) {
    const int rb = min(rows_per_pass, row_hi - r0);
    __syncthreads();
    for (int idx = tid; idx < rb * (Kp / 8); idx += 128) {
      const int m = idx / (Kp / 8), k = (idx - m * (Kp / 8)) * 8;
      const long ar = g.a_rows ? (long)g.a_rows[r0 + m] : (long)(r0 + m);
      const TA* src = A + ar * g.lda;
      TA* dst = As + (size_t)m * Kp + k;
      if (a_vec && k + 8 <= K) {
        if constexpr (sizeof(TA) == 2) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src + k);
        else { *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src + k); *reinterpret_cast<float4*>(dst + 4) = *reinterpret_cast<const float4*>(src + k + 4); }
      } else {
        for (int j = 0; j < 8; ++j) dst[j] = k + j < K ? src[k + j] : (TA)0.f;
      }
    }
    __syncthreads();
    for (int pi = 0; pi < npb / 8; ++pi) {   // this warp's pairs of weight rows
      const int n = n_base + warp * (npb / 4) + pi * 2;
      if (n < g.N) {
        const bool two = n + 1 < g.N;
        const TW* w0 = W + (long)n * g.ldw;
        const TW* w1 = W + (long)(two ? n + 1 : n) * g.ldw;
        float acc[2 * RB];   // [m] row n, [RB + m] row n + 1
#pragma unroll
        for (int m = 0; m < 2 * RB; ++m) acc[m] = 0.f;
        for (int kb = lane * 8; kb < Kp; kb += 4 * 256) {   // four k-steps of both rows in flight
          Raw8<TW> r0[4], r1[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int k = kb + u * 256;
            if (k < Kp) { r0[u].load(w0, k, K, w_vec); r1[u].load(w1, k, K, w_vec); }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int k = kb + u * 256;
            if (k >= Kp) break;
            float f0[8], f1[8];
            r0[u].widen(f0);
            r1[u].widen(f1);
#pragma unroll
            for (int m = 0; m < RB; ++m) {
              if (m < rb) {
                float fa[8];
                load8<TA>(As + (size_t)m * Kp, k, Kp, true, fa);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  acc[m] = fmaf(fa[j], f0[j], acc[m]);
                  acc[RB + m] = fmaf(fa[j], f1[j], acc[RB + m]);
                }
              }
            }
          }
        }
        // 32 sums over 32 lanes in 31 shuffles: each round halves the values a lane holds; lane L ends with value L
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
          const bool upper = (lane & o) != 0;
#pragma unroll
          for (int i = 0; i < o; ++i) {
            const float send = upper ? acc[i] : acc[i + o];
            const float keep = upper ? acc[i + o] : acc[i];
            acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
          }
        }
        // (round o keeps, in a lane whose bit o is set, the upper half of the values it still holds: lane L ends with value L)
        const int m = lane & (RB - 1), which = lane >> 4;   // value L = which * RB + m
        if (m < rb && (which == 0 || two)) {
          float v = acc[0] * g.alpha;
          TC* dst = C + (size_t)(r0 + m) * g.ldc + n + which;
          if (g.epilogue == ANY_EPI_RELU2) {
            v = fmaxf(v, 0.f);
            v = v * v;
          }
          if (g.epilogue == ANY_EPI_ADD) {
            if constexpr (sizeof(TC) == 4) *dst = (TC)((float)*dst + v);
          } else {
            if constexpr (sizeof(TC) == 4) *dst = v;
            else *dst = __float2bfloat16_rn(v);
          }
        }
      }
    }
  }
}

template <typename TA, typename TW, typename TC>
int launch_rows(const AnyGemm& g, int groups, int batch, cudaStream_t s) {
  const int Kp = (g.K + 7) & ~7;
  int rpp = std::min<long>(RB, (long)(96 * 1024) / ((long)Kp * (long)sizeof(TA)));
  if (rpp < 1) return 1;   // a single row does not fit: the caller uses the tile form
  const size_t smem = (size_t)rpp * Kp * sizeof(TA);
  auto kern = gemm_any_rows_kernel<TA, TW, TC>;
  if (smem > 48 * 1024) {
    static B2PerDeviceOnce once;
    if (once.need()) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
  }
  // weight rows per CTA: eight (one pair per warp) while that still gives every SM a few CTAs, more for wide outputs so that
  // the staged rows are reused
  const int other = groups > 0 ? groups : (batch > 0 ? batch : 1);
  int npb = ROWS_NPB;
  while (npb < 64 && (long)((g.N + 2 * npb - 1) / (2 * npb)) * other >= 4 * 148) npb *= 2;
  const dim3 grid((g.N + npb - 1) / npb, groups > 0 ? groups : 1, groups > 0 ? 1 : (batch > 0 ? batch : 1));
  B2_CUDA_OK(b2_launch(kern, grid, dim3(128), smem, s, g, rpp, npb));
  return 0;
}

// ---- few rows, bf16 operands: the weight stream on warp-level MMAs ----
// Above a handful of staged rows the plain-FMA form is bound by its multiply-adds, not by HBM (16 rows cost 256 FMAs per
// 32 weight bytes a lane loads).  Here the weights are the 16 x 16 operand of mma.m16n8k16 and eight token rows the 16 x 8
// one, both loaded from global memory straight into fragment registers with 16-byte loads: inside a 32-wide k chunk lane
// (g, c) = (lane / 4, lane % 4) takes elements [8c, 8c + 8) of weight rows g and g + 8 and of token row g.  An MMA does
// not care which physical k sits behind its logical k as long as both operands agree, so elements 0..3 of the eight feed
// one MMA (logical k 2c, 2c + 1, 2c + 8, 2c + 9) and elements 4..7 the next.  A CTA owns 16 weight rows; its four warps
// take interleaved k chunks (so a weight row is read in 256-byte runs) and their partial tiles are summed in warp order
// through shared memory.  Token rows are re-read by every CTA from L1/L2; the weights are streamed past L1.
__device__ __forceinline__ void mma_16816(float* d, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: eight-row token tiles per pass (rows per pass = 8 * NT); U: k chunks in flight per warp; NW: warps that split K (four when
// the output is wide enough to give every SM several CTAs; eight or sixteen for narrow outputs, whose few CTAs would otherwise
// leave most of an SM's load slots empty -- the choice depends on N, K and the batch count only, never on the rows)
template <typename TC, int NT, int U, int NW>
__global__ void __launch_bounds__(32 * NW) gemm_any_rows_mma_kernel(AnyGemm g) {
  __shared__ float red[NW][NT][32][4];
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, c = lane & 3;
  const bf16* A = reinterpret_cast<const bf16*>(g.A);
  const bf16* W = reinterpret_cast<const bf16*>(g.W);
  TC* C = reinterpret_cast<TC*>(g.C);
  int row_lo, row_hi;
  if (g.group_offsets != nullptr) {   // ragged: blockIdx.y = group
    row_lo = g.group_offsets[blockIdx.y];
    row_hi = g.group_offsets[blockIdx.y + 1];
    if (row_lo >= row_hi) return;
    W += (size_t)blockIdx.y * g.w_bs;
  } else {
    row_lo = 0;
    row_hi = g.M;
    A += (size_t)blockIdx.z * g.a_bs;
    W += (size_t)blockIdx.z * g.w_bs;
    C += (size_t)blockIdx.z * g.c_bs;
  }
  const int K = g.K, n0 = blockIdx.x * 16;
  const bf16* w_lo = W + (long)min(n0 + gq, g.N - 1) * g.ldw + c * 8;       // rows past N are read again and dropped at the store
  const bf16* w_hi = W + (long)min(n0 + gq + 8, g.N - 1) * g.ldw + c * 8;
  const int nchunk = (K + 31) >> 5;
  for (int r0 = row_lo; r0 < row_hi; r0 += 8 * NT) {
    const bf16* tok[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int r = r0 + t * 8 + gq;
      tok[t] = r < row_hi ? A + (g.a_rows ? (long)g.a_rows[r] : (long)r) * g.lda + c * 8 : nullptr;
    }
    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;
    for (int ch0 = warp; ch0 < nchunk; ch0 += NW * U) {
      uint4 wl[U], wh[U], tv[U][NT];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = (ch0 + NW * u) << 5;
        const bool in = k + c * 8 < K;   // K is a multiple of 8: a lane's eight elements are inside or outside together
        wl[u] = in ? ld_stream(w_lo + k) : make_uint4(0, 0, 0, 0);
        wh[u] = in ? ld_stream(w_hi + k) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int t = 0; t < NT; ++t)
          tv[u][t] = (in && tok[t] != nullptr) ? __ldg(reinterpret_cast<const uint4*>(tok[t] + k)) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          mma_16816(acc[t], wl[u].x, wh[u].x, wl[u].y, wh[u].y, tv[u][t].x, tv[u][t].y);
          mma_16816(acc[t], wl[u].z, wh[u].z, wl[u].w, wh[u].w, tv[u][t].z, tv[u][t].w);
        }
    }
    __syncthreads();   // the previous pass has read `red`
#pragma unroll
    for (int t = 0; t < NT; ++t)
      *reinterpret_cast<float4*>(&red[warp][t][lane][0]) = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
    __syncthreads();
    // fragment element i of lane (g, c): weight row g + 8 * (i / 2), token row 2c + (i % 2)
    for (int idx = tid; idx < NT * 128; idx += 32 * NW) {
      const int t = idx >> 7, rem = idx & 127, wr = rem & 15, tk = rem >> 4;   // consecutive threads -> consecutive weight rows
      const int ln = (wr & 7) * 4 + (tk >> 1), i = (wr >> 3) * 2 + (tk & 1);
      const int r = r0 + t * 8 + tk, n = n0 + wr;
      if (r >= row_hi || n >= g.N) continue;
      float v = ((red[0][t][ln][i] + red[1][t][ln][i]) + red[2][t][ln][i]) + red[3][t][ln][i];
#pragma unroll
      for (int w = 4; w < NW; ++w) v += red[w][t][ln][i];
      v *= g.alpha;
      TC* dst = C + (size_t)r * g.ldc + n;
      if (g.epilogue == ANY_EPI_RELU2) {
        v = fmaxf(v, 0.f);
        v = v * v;
      }
      if (g.epilogue == ANY_EPI_ADD) {
        if constexpr (sizeof(TC) == 4) *dst = (TC)((float)*dst + v);
      } else {
        if constexpr (sizeof(TC) == 4) *dst = v;
        else *dst = __float2bfloat16_rn(v);
      }
    }
  }
}

// 16-byte fragment loads need K, both row strides and both bases in multiples of 8 elements
inline bool rows_mma_ok(const AnyGemm& g) {
  return g.K % 8 == 0 && g.lda % 8 == 0 && g.ldw % 8 == 0 && g.a_bs % 8 == 0 && g.w_bs % 8 == 0 &&
         (reinterpret_cast<uintptr_t>(g.A) & 15) == 0 && (reinterpret_cast<uintptr_t>(g.W) & 15) == 0;
}

template <typename TC>
int launch_rows_mma(const AnyGemm& g, int groups, int batch, cudaStream_t s) {
  const dim3 grid((g.N + 15) / 16, groups > 0 ? groups : 1, groups > 0 ? 1 : (batch > 0 ? batch : 1));
  // rows per pass: a ragged group's count is only known on the device (16 covers the usual handful per expert; more rows
  // take more passes over weights that are then in L2)
  const int rows = groups > 0 ? 16 : g.M;
  const long ctas = (long)grid.x * grid.y * grid.z;
  const int nchunk = (g.K + 31) / 32;
  const int nw = (groups > 0 || ctas >= 4 * 148 || nchunk < 32) ? 4 : (ctas >= 2 * 148 || nchunk < 64) ? 8 : 16;
#define ROWS_MMA_LAUNCH(NW)                                                                                        \
  do {                                                                                                             \
    if (rows <= 8) B2_CUDA_OK(b2_launch(gemm_any_rows_mma_kernel<TC, 1, 4, NW>, grid, dim3(32 * NW), 0, s, g));    \
    else if (rows <= 16) B2_CUDA_OK(b2_launch(gemm_any_rows_mma_kernel<TC, 2, 4, NW>, grid, dim3(32 * NW), 0, s, g)); \
    else if (rows <= 32) B2_CUDA_OK(b2_launch(gemm_any_rows_mma_kernel<TC, 4, 2, NW>, grid, dim3(32 * NW), 0, s, g)); \
    else B2_CUDA_OK(b2_launch(gemm_any_rows_mma_kernel<TC, 8, 1, (NW > 8 ? 8 : NW)>, grid, dim3(32 * (NW > 8 ? 8 : NW)), 0, s, g)); /* 48 KB of static shared memory */ \
  } while (0)
  if (nw == 4) ROWS_MMA_LAUNCH(4);
  else if (nw == 8) ROWS_MMA_LAUNCH(8);
  else ROWS_MMA_LAUNCH(16);
#undef ROWS_MMA_LAUNCH
  return 0;
}

// One CTA: tiles of the ragged groups.  group_offsets [G + 1] -> (tile_group, tile_row0, n_tiles).
__global__ void ragged_tiles_kernel(const int* __restrict__ group_offsets, int G, int* __restrict__ tile_group, int* __restrict__ tile_row0,
                                    int* __restrict__ n_tiles, int cap) {
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x != 0) return;
  int n = 0;
  for (int g = 0; g < G; ++g)
    for (int r = group_offsets[g]; r < group_offsets[g + 1] && n < cap; r += BM) {
      tile_group[n] = g;
      tile_row0[n] = r;
      ++n;
    }
  *n_tiles = n;
}

}  // namespace

int any_gemm_tile_rows() { return BM; }
// ragged launches with at most this many rows in all groups together stream the weights and need no tile list
int any_gemm_ragged_rows_limit() {
  static const bool use_rows = [] { const char* e = getenv("B2_ANY_ROWS"); return !(e && *e == '0'); }();
  return use_rows ? 8 * RB : 0;
}

int launch_ragged_tiles(const int* group_offsets, int G, int* tile_group, int* tile_row0, int* n_tiles, int cap, cudaStream_t s) {
  B2_CUDA_OK(b2_launch(ragged_tiles_kernel, dim3(1), dim3(32), 0, s, group_offsets, G, tile_group, tile_row0, n_tiles, cap));
  return 0;
}

int launch_gemm_any(const AnyGemm& g, int a_f32, int w_f32, int c_f32, int batch, int max_tiles, cudaStream_t s, int ragged_rows, int groups) {
  if (g.N <= 0 || g.K <= 0) return 0;
  B2_REQUIRE(g.epilogue != ANY_EPI_ADD || c_f32, "gemm_any: the add epilogue needs an fp32 C");
  {  // few rows: stream the weights (rows of every group counted together for the ragged form: they bound the work per group)
    static const bool use_rows = [] { const char* e = getenv("B2_ANY_ROWS"); return !(e && *e == '0'); }();
    const bool ragged = g.tile_group != nullptr;
    const bool few = (ragged ? (ragged_rows > 0 && ragged_rows <= 8 * RB && groups > 0) : (g.M > 0 && g.M <= 4 * RB)) && g.K <= 16384;
    static const bool use_rows_mma = [] { const char* e = getenv("B2_ANY_ROWS_MMA"); return !(e && *e == '0'); }();  // 0: plain FMAs (cross-check)
    if (use_rows && use_rows_mma && few && !a_f32 && !w_f32 && rows_mma_ok(g))
      return c_f32 ? launch_rows_mma<float>(g, ragged ? groups : 0, batch, s) : launch_rows_mma<bf16>(g, ragged ? groups : 0, batch, s);
    if (use_rows && few && a_f32 == w_f32) {
      int rc = 1;
      if (a_f32 && c_f32) rc = launch_rows<float, float, float>(g, ragged ? groups : 0, batch, s);
      else if (!a_f32 && c_f32) rc = launch_rows<bf16, bf16, float>(g, ragged ? groups : 0, batch, s);
      else if (!a_f32 && !c_f32) rc = launch_rows<bf16, bf16, bf16>(g, ragged ? groups : 0, batch, s);
      if (rc <= 0) return rc;
    }
  }
  dim3 grid;
  if (g.tile_group != nullptr) {
    if (max_tiles <= 0) return 0;
    grid = dim3(max_tiles, (g.N + BN - 1) / BN, 1);
  } else {
    if (g.M <= 0) return 0;
    grid = dim3((g.M + BM - 1) / BM, (g.N + BN - 1) / BN, batch > 0 ? batch : 1);
  }
  static const bool use_mma = [] { const char* e = getenv("B2_ANY_MMA"); return !(e && *e == '0'); }();  // 0: bf16 operands on plain FMAs too (cross-check)
#define GA(TA, TW, TC) B2_CUDA_OK(b2_launch(gemm_any_kernel<TA, TW, TC>, grid, dim3(256), 0, s, g))
  if (a_f32 && w_f32 && c_f32) GA(float, float, float);
  else if (!a_f32 && !w_f32 && use_mma && c_f32) B2_CUDA_OK(b2_launch(gemm_any_mma_kernel<float>, grid, dim3(128), 0, s, g));
  else if (!a_f32 && !w_f32 && use_mma && !c_f32) B2_CUDA_OK(b2_launch(gemm_any_mma_kernel<bf16>, grid, dim3(128), 0, s, g));
  else if (!a_f32 && !w_f32 && c_f32) GA(bf16, bf16, float);
  else if (!a_f32 && !w_f32 && !c_f32) GA(bf16, bf16, bf16);
  else if (a_f32 && !w_f32 && c_f32) GA(float, bf16, float);
  else if (a_f32 && !w_f32 && !c_f32) GA(float, bf16, bf16);
  else {
    b2_set_error("gemm_any: operand type combination (%d, %d, %d) not built", a_f32, w_f32, c_f32);
    return -22;
  }
#undef GA
  return 0;
}

}  // namespace b2
