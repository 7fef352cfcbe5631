// moe_route.cu -- the router of a routed-experts feed-forward, and the bookkeeping that turns its choices into ragged
// groups for gemm_any.cu.
//
// Router (all fp32): z = R x, s = sigmoid(z).  The CHOICE uses s + correction (a per-expert offset that steers load and
// may make a choice score negative); the mixing WEIGHTS use s alone.  Experts are `groups` equal runs of neighbours; a
// group's score is the sum of its two best choice scores and only the `keep` best groups may supply experts (the others
// are out, not zero).  Of the allowed experts the `top` with the best choice scores are taken; their s, divided by their
// sum (+ 1e-20), are the weights.  Ties go to the lower index.
//
// route_permute is a stable counting sort of the (token, choice) pairs by expert: slots of expert e are
// [offsets[e], offsets[e+1]), in (token, choice) order, so the order of the rows inside an expert's GEMM -- and with it
// every sum -- does not depend on the other requests of the batch.  route_combine adds the weighted expert outputs (and the
// mixer branch) onto the fp32 residual stream in choice order.
#include "kernels.h"

namespace b2 {

namespace {

constexpr int RT_WARPS = 4;

template <typename TX>
__global__ void __launch_bounds__(RT_WARPS * 32) route_kernel(const TX* __restrict__ x, const float* __restrict__ router,
                                                              const float* __restrict__ correction, RouteGeom g, int32_t* __restrict__ idx,
                                                              float* __restrict__ weight, int T, int W) {
  extern __shared__ float sm[];  // per warp: s [E], choice [E]
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * RT_WARPS + warp;
  if (t >= T) return;
  const int E = g.experts;
  float* s = sm + (size_t)warp * 2 * E;
  float* ch = s + E;
  const TX* xr = x + (size_t)t * W;
  for (int e = 0; e < E; ++e) {
    const float* rr = router + (size_t)e * W;
    float acc = 0.f;
    for (int i = lane; i < W; i += 32) acc = fmaf((float)xr[i], rr[i], acc);
    acc = warp_sum(acc);
    if (lane == 0) {
      const float sg = 1.0f / (1.0f + expf(-acc));
      s[e] = sg;
      ch[e] = sg + correction[e];
    }
  }
  __syncwarp();
  if (lane != 0) return;
  // groups: score = sum of the two best choice scores; all but the `keep` best are out (choice = -inf).  Ranks are formed
  // from the untouched scores first (a 64-bit mask remembers who is out), then applied.
  const int per = E / g.groups;
  if (g.keep < g.groups) {
    auto group_score = [&](int gi) {
      float b1 = -INFINITY, b2 = -INFINITY;
      for (int e = gi * per; e < (gi + 1) * per; ++e) {
        const float v = ch[e];
        if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
      }
      return per >= 2 ? b1 + b2 : b1;
    };
    unsigned long long out_mask = 0ull;
    for (int gi = 0; gi < g.groups; ++gi) {
      const float my = group_score(gi);
      int beat = 0;  // groups ranked ahead of gi (lower index wins a tie)
      for (int gj = 0; gj < g.groups; ++gj) {
        if (gj == gi) continue;
        const float other = group_score(gj);
        if (other > my || (other == my && gj < gi)) ++beat;
      }
      if (beat >= g.keep) out_mask |= 1ull << gi;
    }
    for (int gi = 0; gi < g.groups; ++gi)
      if ((out_mask >> gi) & 1ull)
        for (int e = gi * per; e < (gi + 1) * per; ++e) ch[e] = -INFINITY;
  }
  float sum = 0.f;
  for (int k = 0; k < g.top; ++k) {
    int best = -1;
    float bv = -INFINITY;
    for (int e = 0; e < E; ++e)
      if (ch[e] > bv) { best = e; bv = ch[e]; }   // -inf = out or already taken; first index wins a tie
    if (best < 0) best = k < E ? k : 0;  // only for rows that hold no numbers (padding rows of a graph bucket): keep the index valid
    idx[(size_t)t * g.top + k] = best;
    weight[(size_t)t * g.top + k] = s[best];
    sum += s[best];
    ch[best] = -INFINITY;
  }
  const float inv = 1.0f / (sum + 1e-20f);
  for (int k = 0; k < g.top; ++k) weight[(size_t)t * g.top + k] *= inv;
}

// one CTA; warp w owns experts w, w + nwarps, ...
__global__ void __launch_bounds__(1024) route_permute_kernel(const int32_t* __restrict__ idx, int npairs, int top, int E,
                                                             int32_t* __restrict__ offsets, int32_t* __restrict__ slot_token,
                                                             int32_t* __restrict__ pair_slot) {
  extern __shared__ int cnt[];  // [E + 1]
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int e = warp; e < E; e += nw) {
    int c = 0;
    for (int p0 = 0; p0 < npairs; p0 += 32) {
      const int p = p0 + lane;
      const bool hit = p < npairs && idx[p] == e;
      c += __popc(__ballot_sync(0xffffffffu, hit));
    }
    if (lane == 0) cnt[e] = c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      const int c = cnt[e];
      cnt[e] = run;
      offsets[e] = run;
      run += c;
    }
    cnt[E] = run;
    offsets[E] = run;
  }
  __syncthreads();
  for (int e = warp; e < E; e += nw) {
    int base = cnt[e];
    for (int p0 = 0; p0 < npairs; p0 += 32) {
      const int p = p0 + lane;
      const bool hit = p < npairs && idx[p] == e;
      const unsigned mask = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int slot = base + __popc(mask & ((1u << lane) - 1u));
        slot_token[slot] = p / top;
        pair_slot[p] = slot;
      }
      base += __popc(mask);
    }
  }
}

__global__ void __launch_bounds__(128) route_combine_kernel(float* __restrict__ h, const float* __restrict__ mix, const float* __restrict__ y,
                                                            const float* __restrict__ weight, const int32_t* __restrict__ pair_slot, int W,
                                                            int top) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < W; i += 128) {
    float acc = mix != nullptr ? mix[(size_t)t * W + i] : 0.f;
    for (int k = 0; k < top; ++k) acc = fmaf(weight[(size_t)t * top + k], y[(size_t)pair_slot[(size_t)t * top + k] * W + i], acc);
    h[(size_t)t * W + i] += acc;
  }
}

}  // namespace

int launch_route(const void* x, int x_f32, const float* router, const float* correction, const RouteGeom& g, int32_t* idx, float* weight,
                 int T, int W, cudaStream_t s) {
  if (T <= 0) return 0;
  B2_REQUIRE(g.experts >= 1 && g.groups >= 1 && g.groups <= 64 && g.experts % g.groups == 0, "route: %d experts do not form %d equal groups", g.experts, g.groups);
  B2_REQUIRE(g.keep >= 1 && g.keep <= g.groups, "route: keep %d outside [1, %d]", g.keep, g.groups);
  B2_REQUIRE(g.top >= 1 && g.top <= g.keep * (g.experts / g.groups), "route: top %d exceeds the %d experts of the kept groups", g.top,
             g.keep * (g.experts / g.groups));
  const size_t smem = (size_t)RT_WARPS * 2 * g.experts * sizeof(float);
  B2_REQUIRE(smem <= 48 * 1024, "route: %d experts need %zu bytes of shared memory", g.experts, smem);
  const dim3 grid((T + RT_WARPS - 1) / RT_WARPS);
  if (x_f32)
    B2_CUDA_OK(b2_launch(route_kernel<float>, grid, dim3(RT_WARPS * 32), smem, s, (const float*)x, router, correction, g, idx, weight, T, W));
  else
    B2_CUDA_OK(b2_launch(route_kernel<bf16>, grid, dim3(RT_WARPS * 32), smem, s, (const bf16*)x, router, correction, g, idx, weight, T, W));
  return 0;
}

int launch_route_permute(const int32_t* idx, int T, int top, int experts, int32_t* offsets, int32_t* slot_token, int32_t* pair_slot,
                         cudaStream_t s) {
  if (T <= 0) return 0;
  const int threads = std::min(1024, std::max(32, experts * 32));
  B2_CUDA_OK(b2_launch(route_permute_kernel, dim3(1), dim3(threads), (size_t)(experts + 1) * sizeof(int), s, idx, T * top, top, experts, offsets,
                       slot_token, pair_slot));
  return 0;
}

int launch_route_combine(float* h, const float* mix, const float* y, const float* weight, const int32_t* pair_slot, int T, int W, int top,
                         cudaStream_t s) {
  if (T <= 0) return 0;
  B2_CUDA_OK(b2_launch(route_combine_kernel, dim3(T), dim3(128), 0, s, h, mix, y, weight, pair_slot, W, top));
  return 0;
}

}  // namespace b2
