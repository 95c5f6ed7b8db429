// Between the query/key/value projection and the attention of a mixer that runs a short causal
// convolution over time on every projected channel:
//
//   u_t   = proj_t + bias                                     (the projection's row, 32-bit)
//   y_t   = sum_j w[c, j] u_(t - taps + 1 + j),  zeros before the request's first token
//   q, k  = rms(y) * weight per head (optional), v = y
//   v    <- (1 - lambda) v + lambda v_first  (optional: v_first are another layer's values of the
//            same tokens; or this layer's v are written out as v_first)
//   q to its rows, k and v into their pages.
//
// The last taps - 1 rows u of every request are its state (32-bit, `[slots, (taps - 1) * C]`, the
// oldest first, zero at a request's start); conv_qkv reads it, conv_state_shift moves it on afterwards.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;

struct ConvIn {
  const float* proj;        // [T, stride]: q | k | v columns, C in all
  long long stride;
  const float* bias;        // [C] or null
  const float* state;       // [slots, state_stride]
  long long state_stride;
  int taps, C;
};

// The convolution's output of channel c for the token at row t, the i-th of its request in this step.
template <typename WT>
__device__ __forceinline__ float conv_at(const ConvIn& in, const WT* __restrict__ w, int t, int i, int slot, int c) {
  const float b = in.bias ? in.bias[c] : 0.f;
  float y = 0.f;
  for (int j = 0; j < in.taps; ++j) {
    const int back = in.taps - 1 - j;          // how many tokens before t
    float u;
    if (back <= i) u = in.proj[(long long)(t - back) * in.stride + c] + b;
    else if (slot >= 0) u = in.state[slot * in.state_stride + (long long)(in.taps - 1 - (back - i)) * in.C + c];
    else u = 0.f;
    y = fmaf(gb::to_float<WT>(w[(size_t)c * in.taps + j]), u, y);
  }
  return y;
}

// The same for a number of taps known when the kernel is compiled. The rows of the step are asked
// for before anything is known of the token's request (`row[j]` may be a row of the request in
// front: it is then dropped for the kept row), so that these loads do not wait for the chain of
// loads that finds the request, its slot and the token's place in it.
template <int TAPS>
struct Taps {
  float row[TAPS], w[TAPS], b;
  __device__ __forceinline__ void ask(const ConvIn& in, const float* __restrict__ conv_w, int t, int c) {
    b = in.bias ? in.bias[c] : 0.f;
#pragma unroll
    for (int j = 0; j < TAPS; ++j) {
      const int back = TAPS - 1 - j;
      row[j] = t >= back ? in.proj[(long long)(t - back) * in.stride + c] : 0.f;
      w[j] = conv_w[(size_t)c * TAPS + j];
    }
  }
  __device__ __forceinline__ float take(const ConvIn& in, int i, int slot, int c) const {
    float y = 0.f;
#pragma unroll
    for (int j = 0; j < TAPS; ++j) {
      const int back = TAPS - 1 - j;
      float u;
      if (back <= i) u = row[j] + b;
      else if (slot >= 0) u = in.state[slot * in.state_stride + (long long)(TAPS - 1 - (back - i)) * in.C + c];
      else u = 0.f;
      y = fmaf(w[j], u, y);
    }
    return y;
  }
};

// grid (tokens, ceil(heads / WARPS)): a warp takes one head of one token (query heads, then key
// heads, then value heads): its lanes convolve the head's channels (every load of the warp is in
// flight at once), the sum of squares crosses the warp, the scaled values are stored. A head's
// channels wait in shared memory between the two (a lane holds any number of them).
// TAPS: the number of taps where it is 1 to 4 (the usual sizes), 0: any number, read from `in`.
template <typename OT, int TAPS>
__global__ void __launch_bounds__(WARPS * 32)
conv_qkv_kernel(ConvIn in, const float* __restrict__ conv_w, OT* __restrict__ q_out, OT* __restrict__ k_pool, OT* __restrict__ v_pool,
                const int32_t* __restrict__ positions, const int32_t* __restrict__ token_req, const int32_t* __restrict__ cu_q,
                const int32_t* __restrict__ slots, const int32_t* __restrict__ block_table, int table_width, int Hq, int Hkv,
                int dim, int vdim, const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                const float* __restrict__ v_first_in, float* __restrict__ v_first_out, float lambda, int page_size) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  extern __shared__ float sm[];            // [WARPS][max(dim, vdim)]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int unit = blockIdx.y * WARPS + warp;
  if (unit >= Hq + 2 * Hkv) return;
  const int t = blockIdx.x;
  const bool is_q = unit < Hq, is_k = !is_q && unit < Hq + Hkv;
  const int head = is_q ? unit : is_k ? unit - Hq : unit - Hq - Hkv;
  const int width = (is_q || is_k) ? dim : vdim;
  const int col = is_q ? head * dim : is_k ? Hq * dim + head * dim : (Hq + Hkv) * dim + head * vdim;
  constexpr int N = TAPS > 0 ? TAPS : 1;
  constexpr int FIRST = 4;                  // channels of a lane whose rows are asked for ahead of everything else
  Taps<N> ahead[FIRST];
  if (TAPS > 0) {
#pragma unroll
    for (int k = 0; k < FIRST; ++k)
      if (lane + 32 * k < width) ahead[k].ask(in, conv_w, t, col + lane + 32 * k);
  }
  const int r = token_req[t];
  const int i = t - cu_q[r];
  const int slot = slots[r];
  const int pos = positions[t];
  const int page = block_table[(size_t)r * table_width + pos / page_size];
  const int in_page = pos % page_size;
  {
    float* buf = sm + (size_t)warp * max(dim, vdim);
    float ss = 0.f;
    if (TAPS > 0) {
#pragma unroll
      for (int k = 0; k < FIRST; ++k) {
        const int c = lane + 32 * k;
        if (c < width) {
          const float y = ahead[k].take(in, i, slot, col + c);
          buf[c] = y;                        // (read back by the lane that wrote it)
          ss += y * y;
        }
      }
      for (int c = lane + 32 * FIRST; c < width; c += 32) {
        Taps<N> one;
        one.ask(in, conv_w, t, col + c);
        const float y = one.take(in, i, slot, col + c);
        buf[c] = y;
        ss += y * y;
      }
    } else {
      for (int c = lane; c < width; c += 32) {
        const float y = conv_at<float>(in, conv_w, t, i, slot, col + c);
        buf[c] = y;
        ss += y * y;
      }
    }
    const float* nw = is_q ? q_w : is_k ? k_w : nullptr;
    const float inv = nw != nullptr ? 1.0f / sqrtf(gb::warp_sum(ss) / (float)width + eps) : 1.f;
    if (is_q) {
      OT* o = q_out + ((size_t)t * Hq + head) * dim;
      for (int c = lane; c < width; c += 32) o[c] = gb::from_float<OT>(nw ? buf[c] * inv * nw[c] : buf[c]);
    } else if (is_k) {
      if (page >= 0) {
        OT* o = k_pool + (((size_t)page * Hkv + head) * page_size + in_page) * dim;
        for (int c = lane; c < width; c += 32) o[c] = gb::from_float<OT>(nw ? buf[c] * inv * nw[c] : buf[c]);
      }
    } else {
      const size_t at = (size_t)t * Hkv * vdim + (size_t)head * vdim;
      OT* o = page >= 0 ? v_pool + (((size_t)page * Hkv + head) * page_size + in_page) * vdim : nullptr;
      for (int c = lane; c < width; c += 32) {
        float v = buf[c];
        if (v_first_out != nullptr) v_first_out[at + c] = v;
        if (v_first_in != nullptr) v = (1.0f - lambda) * v + lambda * v_first_in[at + c];
        if (o != nullptr) o[c] = gb::from_float<OT>(v);
      }
    }
  }
}

// grid (ceil(C / 128), requests): the state after the step, the last taps - 1 rows u of the request.
// A row that this step did not bring comes from the old state; every thread reads all it needs
// before it writes (a channel is one thread's).
__global__ void __launch_bounds__(128)
conv_state_shift_kernel(ConvIn in, float* __restrict__ state, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ slots) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const int c = blockIdx.x * 128 + threadIdx.x;
  if (c >= in.C) return;
  const int r = blockIdx.y;
  const int slot = slots[r];
  if (slot < 0) return;
  const int t0 = cu_q[r], n = cu_q[r + 1] - t0;
  const int keep = in.taps - 1;
  float* s = state + slot * in.state_stride;
  const float b = in.bias ? in.bias[c] : 0.f;
  constexpr int MOST = 15;
  float next[MOST];
#pragma unroll
  for (int k = 0; k < MOST; ++k) {
    if (k < keep) {
      const int back = keep - k;              // row k of the new state lies `back` tokens before the end
      next[k] = back <= n ? in.proj[(long long)(t0 + n - back) * in.stride + c] + b : s[(size_t)(k + n) * in.C + c];
    }
  }
#pragma unroll
  for (int k = 0; k < MOST; ++k)
    if (k < keep) s[(size_t)k * in.C + c] = next[k];
}

}  // namespace

// proj [T, stride]: Hq * dim query, Hkv * dim key and Hkv * vdim value columns; conv_w [C, taps];
// state [slots, state_stride] (read only here). q_w, k_w [dim] 32-bit or null (no norm).
// v_first_in / v_first_out [T, Hkv * vdim] 32-bit, either or both null.
GB_EXPORT int gb_conv_qkv(const float* proj, long long stride, const float* bias, const void* conv_w, int w_dtype, int taps,
                          const float* state, long long state_stride, void* q_out, void* k_pool, void* v_pool, int out_dtype,
                          const int32_t* positions, const int32_t* token_req, const int32_t* cu_q, const int32_t* slots,
                          const int32_t* block_table, int table_width, int T, int Hq, int Hkv, int dim, int vdim,
                          const float* q_w, const float* k_w, float eps, const float* v_first_in, float* v_first_out,
                          float lambda, int page_size, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (taps < 1 || taps > 16) return gb::fail(GB_UNSUPPORTED, "conv_qkv: %d taps (1 to 16)", taps);
  if (taps > 1 && state == nullptr) return gb::fail(GB_BAD_ARGUMENT, "conv_qkv: a convolution needs its state");
  const int C = Hq * dim + Hkv * (dim + vdim);
  const ConvIn in = {proj, stride, bias, state, state_stride, taps, C};
  const size_t smem = (size_t)WARPS * (dim > vdim ? dim : vdim) * sizeof(float);
  if (smem > 48 * 1024) return gb::fail(GB_UNSUPPORTED, "conv_qkv: heads of %d and %d channels", dim, vdim);
  const int units = Hq + 2 * Hkv;
  if ((units + WARPS - 1) / WARPS > 65535) return gb::fail(GB_UNSUPPORTED, "conv_qkv: %d heads", units);
  if (w_dtype != GB_F32) return gb::fail(GB_BAD_ARGUMENT, "conv_qkv: the taps are 32-bit");
  return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
    auto kernel = taps == 1 ? conv_qkv_kernel<OT, 1> : taps == 2 ? conv_qkv_kernel<OT, 2> : taps == 3 ? conv_qkv_kernel<OT, 3>
                : taps == 4 ? conv_qkv_kernel<OT, 4> : conv_qkv_kernel<OT, 0>;
    return gb::check_pdl_launch(
        gb::launch_pdl(kernel, dim3(T, (units + WARPS - 1) / WARPS), dim3(WARPS * 32), smem, stream, dim3(1, 1, 1), in,
                       (const float*)conv_w, (OT*)q_out, (OT*)k_pool, (OT*)v_pool, positions, token_req, cu_q, slots, block_table,
                       table_width, Hq, Hkv, dim, vdim, q_w, k_w, eps, v_first_in, v_first_out, lambda, page_size),
        "conv_qkv");
  });
}

GB_EXPORT int gb_conv_state_shift(const float* proj, long long stride, const float* bias, int taps, int C, float* state,
                                  long long state_stride, const int32_t* cu_q, const int32_t* slots, int R,
                                  cudaStream_t stream) {
  if (R <= 0 || taps <= 1) return GB_OK;
  if (taps > 16) return gb::fail(GB_UNSUPPORTED, "conv_state_shift: %d taps (1 to 16)", taps);
  if (R > 65535) return gb::fail(GB_UNSUPPORTED, "conv_state_shift: %d requests (at most 65535 a step)", R);
  const ConvIn in = {proj, stride, bias, state, state_stride, taps, C};
  return gb::check_pdl_launch(gb::launch_pdl(conv_state_shift_kernel, dim3((C + 127) / 128, R), dim3(128), 0, stream,
                                             dim3(1, 1, 1), in, state, cu_q, slots),
                              "conv_state_shift");
}
