// What a layer needs whose norm comes after the sum, x <- rms(alpha x + sublayer(x)) * w, and two
// small things that its sublayers use. All 32-bit arithmetic.
//
//   post_norm        x <- rms(alpha x + y + row) * w in place on the 32-bit residual (y, row optional), and
//                    the new x rounded to bfloat16 for the sublayer that reads it next; one pass
//   group_gate_mul   x[t, c] <- x[t, c] * sigmoid(gate[t, c / group]): one gate per head
//   xielu            out = a_pos z^2 + z / 2 for z > 0, a_neg (exp(z) - 1 - z) + z / 2 for z <= 0
#include "common.cuh"

GB_DEFINE_LAST_ERROR()

namespace {

inline bool host_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// The block's sum of one value per thread; every thread adds the warps' sums in the same order, so
// the result is the same in every thread and does not depend on the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = gb::warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < warps; ++w) total += scratch[w];
  __syncthreads();
  return total;
}

// One block per token. First pass: v = alpha x + y + row, written over x, and the sum of squares;
// second pass: every thread reads back what it wrote itself, scales and stores.
template <typename WT, bool VEC>
__global__ void __launch_bounds__(256)
post_norm_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ row, float alpha,
                 const WT* __restrict__ w, float eps, __nv_bfloat16* __restrict__ rounded, int d) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  __shared__ float scratch[8];
  const size_t t = blockIdx.x;
  float* xr = x + t * d;
  const float* yr = y ? y + t * d : nullptr;
  float ss = 0.f;
  if (VEC) {
    for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(xr + c);
      v.x *= alpha; v.y *= alpha; v.z *= alpha; v.w *= alpha;
      if (yr) {
        const float4 a = *reinterpret_cast<const float4*>(yr + c);
        v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
      }
      if (row) {
        const float4 a = *reinterpret_cast<const float4*>(row + c);
        v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
      }
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      *reinterpret_cast<float4*>(xr + c) = v;
    }
  } else {
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
      const float v = alpha * xr[c] + (yr ? yr[c] : 0.f) + (row ? row[c] : 0.f);
      ss += v * v;
      xr[c] = v;
    }
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)d + eps);
  __nv_bfloat16* rr = rounded ? rounded + t * d : nullptr;
  if (VEC) {
    for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(xr + c);
      v.x = v.x * inv * gb::to_float<WT>(w[c]);
      v.y = v.y * inv * gb::to_float<WT>(w[c + 1]);
      v.z = v.z * inv * gb::to_float<WT>(w[c + 2]);
      v.w = v.w * inv * gb::to_float<WT>(w[c + 3]);
      *reinterpret_cast<float4*>(xr + c) = v;
      if (rr) {
        gb::store_pair(rr + c, v.x, v.y);
        gb::store_pair(rr + c + 2, v.z, v.w);
      }
    }
  } else {
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
      const float v = xr[c] * inv * gb::to_float<WT>(w[c]);
      xr[c] = v;
      if (rr) rr[c] = __float2bfloat16_rn(v);
    }
  }
}

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

// grid (ceil(n / (PER * 256)), rows): a thread takes PER neighbouring values of a row. VEC: the PER
// values are 16 bytes, lie in one group and rows start on 16 bytes, so they are one load, one gate, one store.
template <typename XT, bool VEC>
__global__ void __launch_bounds__(256)
group_gate_mul_kernel(XT* __restrict__ x, const float* __restrict__ gate, int gate_stride, int n, int group) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  constexpr int PER = 16 / sizeof(XT);
  const size_t t = blockIdx.y;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * PER;
  if (c0 >= n) return;
  XT* xr = x + t * n;
  const float* gr = gate + t * gate_stride;
  if (VEC) {
    const float g = sigmoidf_(gr[c0 / group]);
    XT v[PER];
    *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(xr + c0);
#pragma unroll
    for (int j = 0; j < PER; ++j) v[j] = gb::from_float<XT>(gb::to_float<XT>(v[j]) * g);
    *reinterpret_cast<uint4*>(xr + c0) = *reinterpret_cast<const uint4*>(v);
  } else {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int c = c0 + j;
      if (c < n) xr[c] = gb::from_float<XT>(gb::to_float<XT>(xr[c]) * sigmoidf_(gr[c / group]));
    }
  }
}

__device__ __forceinline__ float xielu(float z, float a_pos, float a_neg) {
  if (z > 0.f) return a_pos * z * z + 0.5f * z;
  return a_neg * (expm1f(z) - z) + 0.5f * z;
}

template <typename IT, typename OT>
__global__ void __launch_bounds__(256)
xielu_kernel(const IT* __restrict__ z, int z_stride, OT* __restrict__ out, int out_stride, int n, float a_pos, float a_neg) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const size_t t = blockIdx.y;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const IT* zr = z + t * z_stride + c0;
  OT* o = out + t * out_stride + c0;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (c0 + j < n) o[j] = gb::from_float<OT>(xielu(gb::to_float<IT>(zr[j]), a_pos, a_neg));
}

}  // namespace

// x [T, d] 32-bit, in place. y [T, d] and row [d]: 32-bit, either may be null. w: the norm's weight.
// rounded (bfloat16 [T, d], optional): the new x rounded.
GB_EXPORT int gb_post_norm(float* x, const float* y, const float* row, float alpha, const void* w, int w_dtype, float eps,
                           void* rounded, int T, int d, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (d < 1) return gb::fail(GB_BAD_ARGUMENT, "post_norm: rows of %d", d);
  const bool vec = d % 4 == 0 && host_aligned16(x) && host_aligned16(y) && host_aligned16(row) &&
                   (reinterpret_cast<uintptr_t>(rounded) & 7) == 0;
  const int threads = d >= 1024 ? 256 : 128;
  return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
    auto kernel = vec ? post_norm_kernel<WT, true> : post_norm_kernel<WT, false>;
    return gb::check_pdl_launch(gb::launch_pdl(kernel, dim3(T), dim3(threads), 0, stream, dim3(1, 1, 1), x, y, row, alpha,
                                               (const WT*)w, eps, (__nv_bfloat16*)rounded, d),
                                "post_norm");
  });
}

// x [T, n] in place; gate [T, n / group] 32-bit logits (a column range of a wider row will do).
GB_EXPORT int gb_group_gate_mul(void* x, int x_dtype, const float* gate, int gate_stride, int T, int n, int group,
                                cudaStream_t stream) {
  if (T <= 0 || n <= 0) return GB_OK;
  if (group < 1 || n % group) return gb::fail(GB_BAD_ARGUMENT, "group_gate_mul: %d values in groups of %d", n, group);
  if (T > 65535) return gb::fail(GB_UNSUPPORTED, "group_gate_mul: %d rows (at most 65535 a call)", T);
  return GB_DISPATCH_DTYPE(x_dtype, XT, [&]() -> int {
    constexpr int PER = 16 / sizeof(XT);
    const dim3 grid((n + PER * 256 - 1) / (PER * 256), T);
    const bool vec = group % PER == 0 && host_aligned16(x);          // (then n, a multiple of group, is one of PER too)
    auto kernel = vec ? group_gate_mul_kernel<XT, true> : group_gate_mul_kernel<XT, false>;
    return gb::check_pdl_launch(gb::launch_pdl(kernel, grid, dim3(256), 0, stream, dim3(1, 1, 1), (XT*)x, gate, gate_stride, n, group),
                                "group_gate_mul");
  });
}

GB_EXPORT int gb_xielu(const void* z, int z_dtype, int z_stride, void* out, int out_dtype, int out_stride, int T, int n,
                       float a_pos, float a_neg, cudaStream_t stream) {
  if (T <= 0 || n <= 0) return GB_OK;
  if (T > 65535) return gb::fail(GB_UNSUPPORTED, "xielu: %d rows (at most 65535 a call)", T);
  const dim3 grid((n + 1023) / 1024, T);
  return GB_DISPATCH_DTYPE(z_dtype, IT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      return gb::check_pdl_launch(gb::launch_pdl(xielu_kernel<IT, OT>, grid, dim3(256), 0, stream, dim3(1, 1, 1), (const IT*)z,
                                                 z_stride, (OT*)out, out_stride, n, a_pos, a_neg),
                                  "xielu");
    });
  });
}
