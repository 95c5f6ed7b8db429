// Routed experts, the plain kernels: a router that picks the `top` largest of E logits per token
// and weighs them by a softmax over the chosen ones, each token's gate/up products against the
// weights of its chosen experts, and the weighted sum of the experts' down products added into the
// residual stream. 32-bit arithmetic; every output is a sum in a fixed order (over k within a
// product, then over a token's choices in the router's order), so a token's result does not depend
// on the rest of the batch.
#include "common.cuh"

namespace {

constexpr int MAX_EXPERTS = 512;
constexpr int MAX_TOP = 32;

// One block per token: its warps share out the experts (z_e = h . W[e] + b[e] in 32-bit, the bias
// 32-bit, each logit one warp's sum in a fixed order), then warp 0 picks the `top` largest in
// descending order (the lower index first among equals); weights = softmax over the chosen logits
// (mode 0), or each chosen expert's own sigmoid(z_e), not renormalized (mode 1), or its share of a
// softmax over all E logits, not renormalized either (mode 2).
template <typename HT, typename WT>
__global__ void __launch_bounds__(256)
route_topk_kernel(const HT* __restrict__ h, const WT* __restrict__ w, const float* __restrict__ bias, int T, int E,
                  int K, int top, int mode, int32_t* __restrict__ ids, float* __restrict__ weights) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  extern __shared__ float sm[];        // z[E], then h[K]
  float* z = sm;
  float* h_s = sm + E;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  const HT* hr = h + (size_t)t * K;
  for (int k = threadIdx.x; k < K; k += blockDim.x) h_s[k] = gb::to_float<HT>(hr[k]);
  __syncthreads();
  for (int e = warp; e < E; e += warps) {
    const WT* wr = w + (size_t)e * K;
    float acc = 0.f;
    for (int k = lane; k < K; k += 32) acc = fmaf(h_s[k], gb::to_float<WT>(wr[k]), acc);
    acc = gb::warp_sum(acc);
    if (lane == 0) z[e] = acc + (bias ? bias[e] : 0.f);
  }
  __syncthreads();
  if (warp != 0) return;
  // the softmax over every expert needs the largest logit and the sum before logits are struck out
  float all_max = -INFINITY, all_sum = 0.f;
  if (mode == 2) {
    for (int e = lane; e < E; e += 32) all_max = fmaxf(all_max, z[e]);
    all_max = gb::warp_max(all_max);
    for (int e = lane; e < E; e += 32) all_sum += expf(z[e] - all_max);
    all_sum = gb::warp_sum(all_sum);
  }
  // `top` rounds of a warp-wide arg-max; a chosen expert's logit is replaced by -inf
  float chosen[MAX_TOP];
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (z[e] > best) { best = z[e]; at = e; }      // the first of equals within a lane
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    chosen[j] = best;
    if (lane == 0) {
      ids[(size_t)t * top + j] = at < E ? at : 0;
      if (at < E) z[at] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0 && mode == 1) {
    for (int j = 0; j < top; ++j) weights[(size_t)t * top + j] = 1.0f / (1.0f + expf(-chosen[j]));
  } else if (lane == 0 && mode == 2) {
    for (int j = 0; j < top; ++j) weights[(size_t)t * top + j] = expf(chosen[j] - all_max) / all_sum;
  } else if (lane == 0) {
    const float largest = chosen[0];
    float sum = 0.f;
    for (int j = 0; j < top; ++j) {
      chosen[j] = expf(chosen[j] - largest);
      sum += chosen[j];
    }
    for (int j = 0; j < top; ++j) weights[(size_t)t * top + j] = chosen[j] / sum;
  }
}

__device__ __forceinline__ float gate_act(int kind, float limit, float g, float u) {
  if (kind == 1) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
  if (kind == 2) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return (g / (1.0f + expf(-1.702f * g))) * (u + 1.0f);
  }
  return (g / (1.0f + expf(-g))) * u;
}

// grid (T, top). act[(t * top + j)][f] = act(gate_e[f] . h_t, up_e[f] . h_t), e = ids[t][j]; the
// expert's weights are [2F, K]: F gate rows, then F up rows. A warp per feature, lanes over k.
// in_scale [T, top] (or null): the pair's factor on the expert's input, expert(s h): both products
// are linear in h, so they are multiplied by s before the activation.
template <typename HT, typename WT, typename OT>
__global__ void __launch_bounds__(128)
moe_gate_up_kernel(const HT* __restrict__ h, const WT* __restrict__ w, const int32_t* __restrict__ ids,
                   OT* __restrict__ act, int top, int F, int K, int kind, float limit,
                   const float* __restrict__ in_scale) {
  extern __shared__ float h_s[];
  const int t = blockIdx.x, j = blockIdx.y;
  for (int k = threadIdx.x; k < K; k += blockDim.x) h_s[k] = gb::to_float<HT>(h[(size_t)t * K + k]);
  __syncthreads();
  const int e = ids[(size_t)t * top + j];
  const float s_in = in_scale ? in_scale[(size_t)t * top + j] : 1.0f;
  const WT* we = w + (size_t)e * 2 * F * K;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int f = warp; f < F; f += 4) {
    const WT* gr = we + (size_t)f * K;
    const WT* ur = we + (size_t)(F + f) * K;
    float g = 0.f, u = 0.f;
    for (int k = lane; k < K; k += 32) {
      g = fmaf(h_s[k], gb::to_float<WT>(gr[k]), g);
      u = fmaf(h_s[k], gb::to_float<WT>(ur[k]), u);
    }
    g = gb::warp_sum(g) * s_in;
    u = gb::warp_sum(u) * s_in;
    if (lane == 0) act[((size_t)t * top + j) * F + f] = gb::from_float<OT>(gate_act(kind, limit, g, u));
  }
}

// One block per token. x[t][n] += alpha * sum_j weights[t][j] * (down_e(j)[n] . act[t][j]); weights null: all one.
template <typename AT, typename WT>
__global__ void __launch_bounds__(256)
moe_down_kernel(const AT* __restrict__ act, const WT* __restrict__ w, const int32_t* __restrict__ ids,
                const float* __restrict__ weights, float* __restrict__ x, int top, int F, int N, float alpha) {
  extern __shared__ float a_s[];        // [top][F]
  const int t = blockIdx.x;
  for (int e = threadIdx.x; e < top * F; e += blockDim.x) a_s[e] = gb::to_float<AT>(act[(size_t)t * top * F + e]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int n = warp; n < N; n += 8) {
    float total = 0.f;
    for (int j = 0; j < top; ++j) {
      const int e = ids[(size_t)t * top + j];
      const WT* wr = w + ((size_t)e * N + n) * F;
      float acc = 0.f;
      for (int f = lane; f < F; f += 32) acc = fmaf(a_s[j * F + f], gb::to_float<WT>(wr[f]), acc);
      total = fmaf(weights ? weights[(size_t)t * top + j] : 1.0f, gb::warp_sum(acc), total);
    }
    if (lane == 0) x[(size_t)t * N + n] = fmaf(alpha, total, x[(size_t)t * N + n]);
  }
}

}  // namespace

GB_EXPORT int gb_route_topk(const void* h, int h_dtype, const void* w, const float* bias, int w_dtype, int T, int E,
                            int K, int top, int mode, int32_t* ids, float* weights, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (mode < 0 || mode > 2) return gb::fail(GB_BAD_ARGUMENT, "route_topk: mode %d", mode);
  if (E < 1 || E > MAX_EXPERTS || top < 1 || top > MAX_TOP || top > E)
    return gb::fail(GB_UNSUPPORTED, "route_topk: %d of %d experts (at most %d of %d)", top, E, MAX_TOP, MAX_EXPERTS);
  const size_t smem = (size_t)(E + K) * sizeof(float);
  if (smem > 200 * 1024) return gb::fail(GB_UNSUPPORTED, "route_topk: width %d", K);
  return GB_DISPATCH_DTYPE(h_dtype, HT, [&]() -> int {
    return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
      if (smem > 48 * 1024) {     // rare (rows beyond 12,000 values): asked for at every such launch
        cudaError_t e = cudaFuncSetAttribute(route_topk_kernel<HT, WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return gb::fail(GB_CUDA_ERROR, "route_topk: %s", cudaGetErrorString(e));
      }
      return gb::check_pdl_launch(
          gb::launch_pdl(route_topk_kernel<HT, WT>, dim3(T), dim3(256), smem, stream,
                         dim3(1, 1, 1), (const HT*)h, (const WT*)w, bias, T, E, K, top, mode, ids, weights),
          "route_topk");
    });
  });
}

GB_EXPORT int gb_moe_gate_up(const void* h, int h_dtype, const void* w, int w_dtype, const int32_t* ids, void* act,
                             int act_dtype, int T, int top, int F, int K, int kind, float limit,
                             const float* in_scale, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if ((size_t)K * sizeof(float) > 48 * 1024) return gb::fail(GB_UNSUPPORTED, "moe_gate_up: width %d", K);
  return GB_DISPATCH_DTYPE(h_dtype, HT, [&]() -> int {
    return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
      return GB_DISPATCH_DTYPE(act_dtype, OT, [&]() -> int {
        moe_gate_up_kernel<HT, WT, OT><<<dim3(T, top), 128, (size_t)K * sizeof(float), stream>>>(
            (const HT*)h, (const WT*)w, ids, (OT*)act, top, F, K, kind, limit, in_scale);
        return gb::check_launch("moe_gate_up");
      });
    });
  });
}

GB_EXPORT int gb_moe_down(const void* act, int act_dtype, const void* w, int w_dtype, const int32_t* ids,
                          const float* weights, float* x, int T, int top, int F, int N, float alpha,
                          cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if ((size_t)top * F * sizeof(float) > 48 * 1024) return gb::fail(GB_UNSUPPORTED, "moe_down: %d x %d activations", top, F);
  return GB_DISPATCH_DTYPE(act_dtype, AT, [&]() -> int {
    return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
      moe_down_kernel<AT, WT><<<T, 256, (size_t)top * F * sizeof(float), stream>>>(
          (const AT*)act, (const WT*)w, ids, weights, x, top, F, N, alpha);
      return gb::check_launch("moe_down");
    });
  });
}
