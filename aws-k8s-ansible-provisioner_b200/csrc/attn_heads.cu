// attn_heads.cu -- softmax attention with per-head keys and values for the layer-list families, any head width, fp32 or
// bf16 cache.  What is optional is a parameter (HeadsGeom), so that one set of kernels serves every mixer of this kind:
//   rotary positions on interleaved pairs of the first rot_dims entries of every query / key head,
//   a short causal convolution over time on every q / k / v channel (the last projected rows of a sequence live in a
//     ring of `taps` rows per sequence slot, indexed by position mod taps: nothing is shifted, a slot that is used again
//     needs no clearing since positions below 0 read as zero, and a token never overwrites a row it reads, so a step
//     that is run twice from the same bookkeeping -- the warm-up ahead of a graph capture -- leaves the same state),
//   q and k heads divided by their root mean square,
//   a linear distance penalty slope_a * (i - j) with slope_a = 2^(-slope_exp (a + 1) / heads),
//   a sliding window that also keeps the first tokens of the sequence,
//   value mixing v <- (1 - lam) v + lam v_first with the values another layer computed for the same token,
//   mixing of the heads' softmax weights by a heads x heads matrix, and a sigmoid gate per head.
//
// Cache: two regions per layer, K rows [kv_heads * dim] and V rows [kv_heads * vdim] per token, in pages of block_size
// tokens; the element type is the engine's operand type.
//
// Arithmetic is fp32 everywhere (angles in fp64 before one rounding): scores, softmax, weights, norms, the convolution and
// its ring.  Only what is stored in a bf16 cache or handed to a bf16 product is rounded.
//
// Kernels:
//   heads_finish      what follows the fused q | k | v (| gate) projection: bias, convolution, rotary or unit-RMS norm,
//                     value mixing, cache row write, fp32 queries
//   conv_tail_store   the ring update, after every token of the step has read the ring
//   heads_attention   one warp per (query token, head) for prompt portions; for a decode step the eight warps of a CTA
//                     split the keys of one (sequence, head) and merge.  Tiles of 32 keys: lane j scores key j, then lane
//                     c accumulates value columns c, c + 32, ...  Key tiles that the window hides are never visited.
//                     With weight mixing ("cross") a query head's weights are applied to the values of EVERY key/value head
//                     (out [heads][kv_heads * vdim], normalised per head), because the mixed output of head a is
//                     sum_b talk[a][b] * (weights of head b applied to the values of a's key/value head)
//   talk_gate         that sum, times the gate, rounded to the operand type
#include "kernels.h"

namespace b2 {

namespace {

template <typename T>
__device__ __forceinline__ float ldf(const T* p);
template <>
__device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ void stf(T* p, float v);
template <>
__device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ void pair_cos_sin(int pos, int i, int dims, float base, float* c, float* s) {
  const double f = exp2(-2.0 * (double)i / (double)dims * log2((double)base));
  double sd, cd;
  sincos((double)pos * f, &sd, &cd);
  *c = (float)cd;
  *s = (float)sd;
}

// One CTA per token.  proj [T][ld] fp32: q (heads * dim) | k (kv_heads * dim) | v (kv_heads * vdim) | anything else.
template <typename TC>
__global__ void __launch_bounds__(128) heads_finish_kernel(const float* __restrict__ proj, int ld, HeadsGeom g, const float* __restrict__ bias,
                                                           const float* __restrict__ conv_w, const float* __restrict__ ring,
                                                           const int32_t* __restrict__ row_seq, const int32_t* __restrict__ row_first,
                                                           const int32_t* __restrict__ positions, const int32_t* __restrict__ slots,
                                                           int vmix_mode, const float* __restrict__ vmix_lambda, float* __restrict__ v_first,
                                                           float* __restrict__ q_out, TC* __restrict__ k_cache, TC* __restrict__ v_cache) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;  // padding row of a decode bucket
  const int pos = positions[t];
  const int nq = g.heads * g.dim, nk = g.kv_heads * g.dim, nv = g.kv_heads * g.vdim, C = nq + nk + nv;
  float* y = sm;            // [C] the token's q | k | v after bias and convolution
  float* cs = sm + C;       // [rot_dims] cos | sin
  const int half = g.rot_dims / 2;
  for (int i = threadIdx.x; i < half; i += 128) pair_cos_sin(pos, i, g.rot_dims, g.rot_base, &cs[i], &cs[half + i]);
  const float* row = proj + (size_t)t * ld;
  if (g.conv_taps > 0) {
    const int taps = g.conv_taps, back = t - row_first[t];
    const float* rg = ring + (size_t)row_seq[t] * taps * C;
    for (int c = threadIdx.x; c < C; c += 128) {
      const float b = bias ? bias[c] : 0.f;
      float acc = 0.f;
      for (int j = 0; j < taps; ++j) {          // y_t = sum_j w[c][j] * u_(t - taps + 1 + j), oldest first
        const int d = taps - 1 - j;             // how far back
        float u = 0.f;
        if (d <= back) u = (row - (size_t)d * ld)[c] + b;
        else if (pos - d >= 0) u = rg[(size_t)((pos - d) % taps) * C + c];
        acc = fmaf(conv_w[(size_t)c * taps + j], u, acc);
      }
      y[c] = acc;
    }
  } else {
    for (int c = threadIdx.x; c < C; c += 128) y[c] = row[c] + (bias ? bias[c] : 0.f);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // q and k heads: one warp per head
  for (int hh = warp; hh < g.heads + g.kv_heads; hh += 4) {
    float* v = y + (size_t)hh * g.dim;  // q heads first, then k heads: both g.dim wide
    if (g.unit_qk) {
      float ss = 0.f;
      for (int d = lane; d < g.dim; d += 32) ss = fmaf(v[d], v[d], ss);
      ss = warp_sum(ss);
      const float r = 1.0f / sqrtf(ss / (float)g.dim + g.eps);
      for (int d = lane; d < g.dim; d += 32) v[d] *= r;
    }
    for (int p = lane; p < half; p += 32) {
      const float a = v[2 * p], b = v[2 * p + 1];
      v[2 * p] = a * cs[p] - b * cs[half + p];
      v[2 * p + 1] = b * cs[p] + a * cs[half + p];
    }
  }
  // values
  if (vmix_mode != 0) {
    float* vf = v_first + (size_t)t * nv;
    if (vmix_mode == 1) {
      for (int c = threadIdx.x; c < nv; c += 128) vf[c] = y[nq + nk + c];
    } else {
      const float lam = *vmix_lambda;
      for (int c = threadIdx.x; c < nv; c += 128) y[nq + nk + c] = (1.0f - lam) * y[nq + nk + c] + lam * vf[c];
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < nq; c += 128) q_out[(size_t)t * nq + c] = y[c];
  TC* kr = k_cache + (size_t)slot * nk;
  for (int c = threadIdx.x; c < nk; c += 128) stf(kr + c, y[nq + c]);
  TC* vr = v_cache + (size_t)slot * nv;
  for (int c = threadIdx.x; c < nv; c += 128) stf(vr + c, y[nq + nk + c]);
}

__global__ void __launch_bounds__(128) conv_tail_store_kernel(const float* __restrict__ proj, int ld, int C, int taps,
                                                              const float* __restrict__ bias, float* __restrict__ ring,
                                                              const int32_t* __restrict__ row_seq, const int32_t* __restrict__ row_end,
                                                              const int32_t* __restrict__ positions, const int32_t* __restrict__ slots) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  if (slots[t] < 0) return;
  if (row_end[t] - 1 - t >= taps) return;  // a later token of the same portion owns this ring row
  float* dst = ring + ((size_t)row_seq[t] * taps + positions[t] % taps) * C;
  const float* row = proj + (size_t)t * ld;
  for (int c = threadIdx.x; c < C; c += 128) dst[c] = row[c] + (bias ? bias[c] : 0.f);
}

constexpr int HA_WARPS = 8;

// Visible key tiles of query position i: tiles [0, nA) cover the kept first tokens, tiles [tB, i / 32] the window.
struct TileRange {
  int nA, tB, total;
};
__device__ __forceinline__ TileRange visible_tiles(int i, int window, int keep_first) {
  TileRange r;
  const int last = i >> 5;
  if (window <= 0) {
    r.nA = 0; r.tB = 0; r.total = last + 1;
    return r;
  }
  const int lo = max(i - window + 1, 0);
  const int endA = min(keep_first, lo);  // kept keys below the window
  r.nA = (endA + 31) >> 5;
  r.tB = max(lo >> 5, r.nA);
  r.total = r.nA + (last - r.tB + 1);
  return r;
}

// NV = ceil(value columns / 32).  DECODE: a CTA is one (sequence, head), its warps take the visible key tiles round robin;
// else a CTA is eight query tokens of one tile and one head, a warp per token.
template <typename TC, typename TO, int NV, bool DECODE>
__global__ void __launch_bounds__(HA_WARPS * 32) heads_attention_kernel(const float* __restrict__ q, const TC* __restrict__ k_cache,
                                                                        const TC* __restrict__ v_cache, HeadsGeom g,
                                                                        const int32_t* __restrict__ block_table, int bt_stride, int block_size,
                                                                        const PrefillTile* __restrict__ tiles, const int32_t* __restrict__ positions,
                                                                        const int32_t* __restrict__ seq_lens, TO* __restrict__ out) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int a = blockIdx.y, kvh = a / (g.heads / g.kv_heads);
  const int D = g.dim, krow = g.kv_heads * g.dim, vrow = g.kv_heads * g.vdim;
  const int VW = g.cross ? vrow : g.vdim, voff = g.cross ? 0 : kvh * g.vdim;
  int t, pos, bt_row;
  bool live;
  if (DECODE) {
    t = blockIdx.x;
    bt_row = t;
    live = seq_lens[t] > 0;
    pos = live ? positions[t] : 0;
  } else {
    const PrefillTile tl = tiles[blockIdx.x >> 3];
    const int r = ((blockIdx.x & 7) << 3) + warp;
    live = r < tl.nrows;
    t = tl.q_row0 + r;
    pos = tl.q_pos0 + r;
    bt_row = tl.bt_row;
    if (((blockIdx.x & 7) << 3) >= tl.nrows) return;
  }
  float* qs = sm + (DECODE ? 0 : (size_t)warp * D);
  if (live) {
    const float* qr = q + ((size_t)t * g.heads + a) * D;
    if (DECODE) {
      for (int d = threadIdx.x; d < D; d += HA_WARPS * 32) qs[d] = qr[d];
    } else {
      for (int d = lane; d < D; d += 32) qs[d] = qr[d];
    }
  }
  if (DECODE) __syncthreads();
  else __syncwarp();
  const float slope = g.slopes ? (float)exp2(-(double)g.slope_exp * (double)(a + 1) / (double)g.heads) : 0.f;
  float m = -INFINITY, l = 0.f, acc[NV];
#pragma unroll
  for (int n = 0; n < NV; ++n) acc[n] = 0.f;
  if (live) {
    const TileRange tr = visible_tiles(pos, g.window, g.keep_first);
    const int32_t* bt = block_table + (size_t)bt_row * bt_stride;
    const int lo = g.window > 0 ? pos - g.window + 1 : 0;
    for (int vi = DECODE ? warp : 0; vi < tr.total; vi += DECODE ? HA_WARPS : 1) {
      const int tile = vi < tr.nA ? vi : tr.tB + (vi - tr.nA);
      const int j = (tile << 5) + lane;
      const bool vis = j <= pos && (g.window <= 0 || j >= lo || j < g.keep_first);
      float s = -INFINITY;
      size_t slot = 0;
      if (vis) {
        slot = (size_t)bt[j / block_size] * block_size + j % block_size;
        const TC* kr = k_cache + slot * krow + (size_t)kvh * D;
        float dot = 0.f;
        for (int d = 0; d < D; ++d) dot = fmaf(qs[d], ldf(kr + d), dot);
        s = dot * g.scale - slope * (float)(pos - j);
      }
      const float mt = warp_max(s);  // finite: a visited tile holds at least one visible key
      const float mn = fmaxf(m, mt);
      const float corr = expf(m - mn);  // exp(-inf) = 0 on the first tile
      const float p = vis ? expf(s - mn) : 0.f;
      l = l * corr + warp_sum(p);
#pragma unroll
      for (int n = 0; n < NV; ++n) acc[n] *= corr;
      m = mn;
      unsigned mask = __ballot_sync(0xffffffffu, vis);
      while (mask) {
        const int jj = __ffs(mask) - 1;
        mask &= mask - 1;
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        const size_t sj = __shfl_sync(0xffffffffu, (unsigned long long)slot, jj);
        const TC* vr = v_cache + sj * vrow + voff;
#pragma unroll
        for (int n = 0; n < NV; ++n) {
          const int c = lane + 32 * n;
          if (c < VW) acc[n] = fmaf(pj, ldf(vr + c), acc[n]);
        }
      }
    }
  }
  TO* orow = out + ((size_t)t * g.heads + a) * VW;
  if (!DECODE) {
    if (!live) return;
    const float inv = 1.0f / l;
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      const int c = lane + 32 * n;
      if (c < VW) stf(orow + c, acc[n] * inv);
    }
    return;
  }
  // merge the warps' partial sums in warp order
  float* ms = sm + D;            // [8] maxima, [8] sums, [8][VW] accumulators
  float* ls = ms + HA_WARPS;
  float* as = ls + HA_WARPS;
  if (lane == 0) {
    ms[warp] = m;
    ls[warp] = l;
  }
#pragma unroll
  for (int n = 0; n < NV; ++n) {
    const int c = lane + 32 * n;
    if (c < VW) as[(size_t)warp * VW + c] = acc[n];
  }
  __syncthreads();
  float M = -INFINITY;
  for (int w = 0; w < HA_WARPS; ++w) M = fmaxf(M, ms[w]);
  float L = 0.f;
  float f[HA_WARPS];
  for (int w = 0; w < HA_WARPS; ++w) {
    f[w] = ms[w] == -INFINITY ? 0.f : expf(ms[w] - M);
    L = fmaf(ls[w], f[w], L);
  }
  const float inv = live && L > 0.f ? 1.0f / L : 0.f;
  for (int c = threadIdx.x; c < VW; c += HA_WARPS * 32) {
    float o = 0.f;
    for (int w = 0; w < HA_WARPS; ++w) o = fmaf(as[(size_t)w * VW + c], f[w], o);
    stf(orow + c, o * inv);
  }
}

// out[t][a][d] = sigmoid(gate[t][a]) * sum_b talk[a][b] * cross[t][b][kv(a) * vdim + d]
template <typename TX>
__global__ void __launch_bounds__(128) talk_gate_kernel(const float* __restrict__ cross, const float* __restrict__ talk,
                                                        const float* __restrict__ gate, int gate_ld, TX* __restrict__ out, int heads,
                                                        int kv_heads, int vdim) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, rep = heads / kv_heads, vrow = kv_heads * vdim;
  const float* cr = cross + (size_t)t * heads * vrow;
  for (int i = threadIdx.x; i < heads * vdim; i += 128) {
    const int a = i / vdim, d = i - a * vdim, col = (a / rep) * vdim + d;
    float o = 0.f;
    for (int b = 0; b < heads; ++b) o = fmaf(talk[a * heads + b], cr[(size_t)b * vrow + col], o);
    const float gl = gate ? gate[(size_t)t * gate_ld + a] : 0.f;
    const float gv = gate ? 1.0f / (1.0f + expf(-gl)) : 1.0f;
    stf(out + (size_t)t * heads * vdim + i, o * gv);
  }
}

template <typename TC, typename TO, bool DECODE>
int launch_attention_nv(int nv, dim3 grid, size_t smem, cudaStream_t s, const float* q, const TC* k, const TC* v, const HeadsGeom& g,
                        const int32_t* bt, int bt_stride, int block_size, const PrefillTile* tiles, const int32_t* positions,
                        const int32_t* seq_lens, TO* out) {
#define HA_CASE(NVV)                                                                                                                   \
  if (nv <= NVV) {                                                                                                                     \
    auto kern = heads_attention_kernel<TC, TO, NVV, DECODE>;                                                                           \
    if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));              \
    B2_CUDA_OK(b2_launch(kern, grid, dim3(HA_WARPS * 32), smem, s, q, k, v, g, bt, bt_stride, block_size, tiles, positions, seq_lens, out)); \
    return 0;                                                                                                                          \
  }
  HA_CASE(1) HA_CASE(2) HA_CASE(4) HA_CASE(8) HA_CASE(16) HA_CASE(32)
#undef HA_CASE
  b2_set_error("heads_attention: %d value columns per query head exceed 1024", nv * 32);
  return -22;
}

template <typename TC, typename TO>
int launch_attention_t(const float* q, const void* k, const void* v, const HeadsGeom& g, const int32_t* bt, int bt_stride, int block_size,
                       const PrefillTile* tiles, int ntiles, const int32_t* positions, const int32_t* seq_lens, void* out, int T,
                       cudaStream_t s) {
  const int VW = g.cross ? g.kv_heads * g.vdim : g.vdim, nv = (VW + 31) / 32;
  if (tiles != nullptr) {
    const size_t smem = (size_t)HA_WARPS * g.dim * sizeof(float);
    return launch_attention_nv<TC, TO, false>(nv, dim3(ntiles * 8, g.heads), smem, s, q, (const TC*)k, (const TC*)v, g, bt, bt_stride,
                                              block_size, tiles, positions, seq_lens, (TO*)out);
  }
  const size_t smem = ((size_t)g.dim + 2 * HA_WARPS + (size_t)HA_WARPS * VW) * sizeof(float);
  return launch_attention_nv<TC, TO, true>(nv, dim3(T, g.heads), smem, s, q, (const TC*)k, (const TC*)v, g, bt, bt_stride, block_size,
                                           nullptr, positions, seq_lens, (TO*)out);
}

}  // namespace

int launch_heads_finish(const float* proj, int ld, const HeadsGeom& g, const float* bias, const float* conv_w, float* ring,
                        const int32_t* row_seq, const int32_t* row_first, const int32_t* row_end, const int32_t* positions,
                        const int32_t* slots, int vmix_mode, const float* vmix_lambda, float* v_first, float* q_out, void* k_cache,
                        void* v_cache, int cache_f32, int T, cudaStream_t s) {
  if (T <= 0) return 0;
  B2_REQUIRE(g.rot_dims >= 0 && g.rot_dims <= g.dim && g.rot_dims % 2 == 0, "heads_finish: rot dims %d must be even and <= dim %d", g.rot_dims,
             g.dim);
  B2_REQUIRE(g.conv_taps == 0 || (conv_w && ring && row_seq && row_first && row_end), "heads_finish: the convolution needs its weights and state");
  B2_REQUIRE(vmix_mode == 0 || v_first != nullptr, "heads_finish: value mixing needs the first layer's values");
  const int C = g.heads * g.dim + g.kv_heads * (g.dim + g.vdim);
  const size_t smem = ((size_t)C + std::max(g.rot_dims, 2)) * sizeof(float);
  B2_REQUIRE(smem <= 200 * 1024, "heads_finish: q | k | v row of %d numbers exceeds shared memory", C);
  if (cache_f32) {
    auto kern = heads_finish_kernel<float>;
    if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    B2_CUDA_OK(b2_launch(kern, dim3(T), dim3(128), smem, s, proj, ld, g, bias, conv_w, (const float*)ring, row_seq, row_first, positions, slots,
                         vmix_mode, vmix_lambda, v_first, q_out, (float*)k_cache, (float*)v_cache));
  } else {
    auto kern = heads_finish_kernel<bf16>;
    if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    B2_CUDA_OK(b2_launch(kern, dim3(T), dim3(128), smem, s, proj, ld, g, bias, conv_w, (const float*)ring, row_seq, row_first, positions, slots,
                         vmix_mode, vmix_lambda, v_first, q_out, (bf16*)k_cache, (bf16*)v_cache));
  }
  if (g.conv_taps > 1)
    B2_CUDA_OK(b2_launch(conv_tail_store_kernel, dim3(T), dim3(128), 0, s, proj, ld, C, g.conv_taps, bias, ring, row_seq, row_end, positions, slots));
  return 0;
}

int launch_heads_attention(const float* q, const void* k_cache, const void* v_cache, int cache_f32, const HeadsGeom& g,
                           const int32_t* block_table, int bt_stride, int block_size, const PrefillTile* tiles, int ntiles,
                           const int32_t* positions, const int32_t* seq_lens, void* out, int out_f32, int T, cudaStream_t s) {
  if (T <= 0 || (tiles != nullptr && ntiles <= 0)) return 0;
  B2_REQUIRE(g.heads >= 1 && g.kv_heads >= 1 && g.heads % g.kv_heads == 0, "heads_attention: %d query heads over %d key/value heads", g.heads,
             g.kv_heads);
  B2_REQUIRE(!g.cross || out_f32, "heads_attention: the per-head sums that are mixed afterwards are fp32");
  if (cache_f32) {
    B2_REQUIRE(out_f32, "heads_attention: an fp32 cache goes with fp32 operands");
    return launch_attention_t<float, float>(q, k_cache, v_cache, g, block_table, bt_stride, block_size, tiles, ntiles, positions, seq_lens, out, T, s);
  }
  if (out_f32)
    return launch_attention_t<bf16, float>(q, k_cache, v_cache, g, block_table, bt_stride, block_size, tiles, ntiles, positions, seq_lens, out, T, s);
  return launch_attention_t<bf16, bf16>(q, k_cache, v_cache, g, block_table, bt_stride, block_size, tiles, ntiles, positions, seq_lens, out, T, s);
}

int launch_talk_gate(const float* cross, const float* talk, const float* gate, int gate_ld, void* out, int out_f32, int heads, int kv_heads,
                     int vdim, int T, cudaStream_t s) {
  if (T <= 0) return 0;
  if (out_f32) B2_CUDA_OK(b2_launch(talk_gate_kernel<float>, dim3(T), dim3(128), 0, s, cross, talk, gate, gate_ld, (float*)out, heads, kv_heads, vdim));
  else B2_CUDA_OK(b2_launch(talk_gate_kernel<bf16>, dim3(T), dim3(128), 0, s, cross, talk, gate, gate_ld, (bf16*)out, heads, kv_heads, vdim));
  return 0;
}

}  // namespace b2
