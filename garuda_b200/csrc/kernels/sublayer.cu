// Kernels around a sublayer whose output, not its input, is normed, and for attention whose
// queries and keys are normed per head before they are rotated. All arithmetic is 32-bit.
//
//   qk_norm_rope_append  a projected row -> queries (RMS norm per head with a weight per head and
//                        channel, rotation of the first channels) to q_out; keys (the same, one
//                        weight for all heads) and values into their pages; the values may be the
//                        keys' own columns as projected (before norm and rotation)
//   gate_mul             x <- x * act(gate), act = sigmoid | silu, the gate's logits 32-bit
//   unary_act            out = act(z), act = relu^2 | tanh
//   sublayer_merge       y = alpha * sum_b rms(y_b) * w_b   (or y = y_0)
//                        y <- y * sigmoid(gate + bias)      (optional)
//                        x <- x + rms(y) * w                (or out = y)
//                        h = x rounded to bfloat16          (optional: the next sublayer's input)
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

constexpr int QK_MAX_DIM = 256;

// One block per token, a warp per head in turn (queries, then keys, then values).
template <typename OT>
__global__ void __launch_bounds__(256)
qk_norm_rope_append_kernel(const float* __restrict__ src, int row_stride, int q_col, int k_col, int v_col,
                           OT* __restrict__ q_out, OT* __restrict__ k_pool, OT* __restrict__ v_pool,
                           const int32_t* __restrict__ positions, const int32_t* __restrict__ token_req,
                           const int32_t* __restrict__ block_table, int table_width, int Hq, int Hkv, int dim, int vdim,
                           const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                           const float* __restrict__ inv_freq, int interleaved, int page_size) {
  __shared__ float sin_s[QK_MAX_DIM / 2], cos_s[QK_MAX_DIM / 2];
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = dim >> 1;
  const bool rotate = inv_freq != nullptr;
  if (rotate)
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sin_s[i], &cos_s[i]);
  long long cache_row = -1;
  if (Hkv > 0) {
    const int page = block_table[(size_t)token_req[t] * table_width + pos / page_size];
    if (page >= 0) cache_row = (long long)page * Hkv;       // no page behind this position: nothing is stored
  }
  __syncthreads();
  const float* row = src + (size_t)t * row_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  // every head of the row starts on 8 bytes (the head width is even)
  const bool paired = interleaved && ((row_stride | q_col | k_col) & 1) == 0 && (reinterpret_cast<uintptr_t>(src) & 7) == 0 &&
                      ((reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_pool)) & (2 * sizeof(OT) - 1)) == 0;
  for (int head = warp; head < Hq + Hkv; head += warps) {
    const bool is_q = head < Hq;
    if (!is_q && cache_row < 0) continue;
    const float* s = row + (is_q ? q_col + head * dim : k_col + (head - Hq) * dim);
    const float* w = is_q ? (q_w ? q_w + (size_t)head * dim : nullptr) : k_w;
    const bool normed = is_q ? q_w != nullptr : k_w != nullptr;
    float inv = 1.0f;
    if (normed) {
      float ss = 0.f;
      for (int c = lane; c < dim; c += 32) ss = fmaf(s[c], s[c], ss);
      inv = 1.0f / sqrtf(gb::warp_sum(ss) / (float)dim + eps);
    }
    OT* dst = is_q ? q_out + ((size_t)t * Hq + head) * dim
                   : k_pool + ((cache_row + (head - Hq)) * page_size + (pos % page_size)) * dim;
    if (paired) {        // neighbours rotate together: one 8-byte load and one store for the two
      for (int i = lane; i < half; i += 32) {
        const float2 ab = *reinterpret_cast<const float2*>(s + 2 * i);
        float a = ab.x, b = ab.y;
        if (normed) a = (a * inv) * w[2 * i], b = (b * inv) * w[2 * i + 1];
        if (rotate) {
          const float ra = a * cos_s[i] - b * sin_s[i], rb = b * cos_s[i] + a * sin_s[i];
          a = ra, b = rb;
        }
        gb::store_pair(dst + 2 * i, a, b);
      }
      continue;
    }
    for (int i = lane; i < half; i += 32) {
      const int ia = interleaved ? 2 * i : i;
      const int ib = interleaved ? 2 * i + 1 : i + half;
      float a = s[ia], b = s[ib];
      if (normed) a = (a * inv) * w[ia], b = (b * inv) * w[ib];
      if (rotate) {
        const float ra = a * cos_s[i] - b * sin_s[i], rb = b * cos_s[i] + a * sin_s[i];
        a = ra, b = rb;
      }
      dst[ia] = gb::from_float<OT>(a);
      dst[ib] = gb::from_float<OT>(b);
    }
  }
  if (cache_row >= 0) {
    const float* vs = row + v_col;
    for (int e = threadIdx.x; e < Hkv * vdim; e += blockDim.x) {
      const int head = e / vdim, c = e % vdim;
      v_pool[((cache_row + head) * page_size + (pos % page_size)) * vdim + c] = gb::from_float<OT>(vs[e]);
    }
  }
}

enum { ACT_SIGMOID = 0, ACT_SILU = 1, ACT_RELU2 = 2, ACT_TANH = 3 };

__device__ __forceinline__ float act(float z, int kind) {
  switch (kind) {
    case ACT_SIGMOID: return sigmoidf_(z);
    case ACT_SILU: return z * sigmoidf_(z);
    case ACT_RELU2: { const float r = fmaxf(z, 0.f); return r * r; }
    default: return tanhf(z);
  }
}

// grid (ceil(n / (4 * 256)), rows): a thread takes four neighbouring values of one row (VEC: rows start on
// 16 bytes and n is a multiple of four, so the four are one load), else one value at a time.
template <typename XT, bool VEC>
__global__ void __launch_bounds__(256)
gate_mul_kernel(XT* __restrict__ x, const float* __restrict__ gate, int gate_stride, int n, int kind) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const size_t t = blockIdx.y;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c0 >= n) return;
  XT* xr = x + t * n + c0;
  const float* gr = gate + t * gate_stride + c0;
  if (VEC) {
    const float4 g = *reinterpret_cast<const float4*>(gr);
    const float gs[4] = {g.x, g.y, g.z, g.w};
    XT v[4];
    if (sizeof(XT) == 2) *reinterpret_cast<uint2*>(v) = *reinterpret_cast<const uint2*>(xr);
    else *reinterpret_cast<float4*>(v) = *reinterpret_cast<const float4*>(xr);
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = gb::from_float<XT>(gb::to_float<XT>(v[j]) * act(gs[j], kind));
    if (sizeof(XT) == 2) *reinterpret_cast<uint2*>(xr) = *reinterpret_cast<const uint2*>(v);
    else *reinterpret_cast<float4*>(xr) = *reinterpret_cast<const float4*>(v);
  } else {
    for (int j = 0; j < 4 && c0 + j < n; ++j) xr[j] = gb::from_float<XT>(gb::to_float<XT>(xr[j]) * act(gr[j], kind));
  }
}

template <typename IT, typename OT>
__global__ void __launch_bounds__(256)
unary_act_kernel(const IT* __restrict__ z, int z_stride, OT* __restrict__ out, int out_stride, int n, int kind) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const size_t t = blockIdx.y;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const IT* zr = z + t * z_stride + c0;
  OT* o = out + t * out_stride + c0;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (c0 + j < n) o[j] = gb::from_float<OT>(act(gb::to_float<IT>(zr[j]), kind));
}

constexpr int MAX_BRANCHES = 4;
struct Branches {
  const float* y[MAX_BRANCHES];
  const float* w[MAX_BRANCHES];
  int n;
};

// Sums of up to MAX_BRANCHES values over the block at once; every thread adds the warps' sums in the
// same order.
template <int N>
__device__ __forceinline__ void block_sums(float (&v)[N], float* red) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = gb::warp_sum(v[i]);
  __syncthreads();                  // `red` may still be read from the call before
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) red[warp * N + i] = v[i];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < N; ++i) {
    float total = 0.f;
    for (int w = 0; w < warps; ++w) total += red[w * N + i];
    v[i] = total;
  }
}

// One block per token. A thread owns the channels c with (c / 4) % blockDim.x == threadIdx.x (four
// neighbours at a time; VEC: as one 16-byte access). Pass 1: every branch's sum of squares. Pass 2: the
// merged, gated row (kept in shared memory) and its sum of squares. Pass 3: the residual and its rounded copy.
template <bool VEC>
__global__ void __launch_bounds__(256)
sublayer_merge_kernel(Branches br, float alpha, float branch_eps, const float* __restrict__ gate, int gate_stride,
                      const float* __restrict__ gate_bias, const float* __restrict__ w, float eps, float* __restrict__ x,
                      float* __restrict__ out, __nv_bfloat16* __restrict__ rounded, int d) {
  extern __shared__ __align__(16) float rowbuf[];       // [d rounded up to four]
  __shared__ float red[8 * MAX_BRANCHES];
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const size_t t = blockIdx.x;
  const bool merged = br.w[0] != nullptr;
  auto load4 = [&](const float* p, int c, float (&v)[4]) {
    if (VEC) {
      const float4 q = *reinterpret_cast<const float4*>(p + c);
      v[0] = q.x, v[1] = q.y, v[2] = q.z, v[3] = q.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = c + j < d ? p[c + j] : 0.f;
    }
  };
  float inv_b[MAX_BRANCHES] = {1.f, 1.f, 1.f, 1.f};
  if (merged) {
    float ss[MAX_BRANCHES] = {0.f, 0.f, 0.f, 0.f};
    for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
#pragma unroll
      for (int b = 0; b < MAX_BRANCHES; ++b) {
        if (b >= br.n) break;
        float v[4];
        load4(br.y[b] + t * d, c, v);
#pragma unroll
        for (int j = 0; j < 4; ++j) ss[b] = fmaf(v[j], v[j], ss[b]);
      }
    }
    block_sums(ss, red);
#pragma unroll
    for (int b = 0; b < MAX_BRANCHES; ++b) inv_b[b] = alpha / sqrtf(ss[b] / (float)d + branch_eps);
  }
  float sq[1] = {0.f};
  for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
    float y[4] = {0.f, 0.f, 0.f, 0.f};
    if (merged) {
#pragma unroll
      for (int b = 0; b < MAX_BRANCHES; ++b) {
        if (b >= br.n) break;
        float v[4], wb[4];
        load4(br.y[b] + t * d, c, v);
        load4(br.w[b], c, wb);
#pragma unroll
        for (int j = 0; j < 4; ++j) y[j] = fmaf(v[j] * inv_b[b], wb[j], y[j]);
      }
    } else {
      load4(br.y[0] + t * d, c, y);
    }
    if (gate != nullptr) {
      float g[4], gbias[4] = {0.f, 0.f, 0.f, 0.f};
      if (VEC) load4(gate + t * gate_stride, c, g);
      else {
#pragma unroll
        for (int j = 0; j < 4; ++j) g[j] = c + j < d ? gate[t * gate_stride + c + j] : 0.f;
      }
      if (gate_bias != nullptr) load4(gate_bias, c, gbias);
#pragma unroll
      for (int j = 0; j < 4; ++j) y[j] *= sigmoidf_(g[j] + gbias[j]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (c + j < d) {
        if (x == nullptr) out[t * d + c + j] = y[j];
        else rowbuf[c + j] = y[j];
        sq[0] = fmaf(y[j], y[j], sq[0]);
      }
    }
  }
  if (x == nullptr) return;
  block_sums(sq, red);
  const float inv = 1.0f / sqrtf(sq[0] / (float)d + eps);
  for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
    float xv[4], wv[4];
    load4(x + t * d, c, xv);
    load4(w, c, wv);
#pragma unroll
    for (int j = 0; j < 4; ++j) xv[j] += (rowbuf[c + j] * inv) * wv[j];      // a thread reads back what it wrote itself
    if (VEC) {
      *reinterpret_cast<float4*>(x + t * d + c) = make_float4(xv[0], xv[1], xv[2], xv[3]);
      if (rounded != nullptr) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(xv[0], xv[1]), hi = __floats2bfloat162_rn(xv[2], xv[3]);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(rounded + t * d + c) = packed;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c + j < d) {
          x[t * d + c + j] = xv[j];
          if (rounded != nullptr) rounded[t * d + c + j] = __float2bfloat16_rn(xv[j]);
        }
    }
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

GB_EXPORT int gb_qk_norm_rope_append(const float* src, int row_stride, int q_col, int k_col, int v_col, void* q_out,
                                     void* k_pool, void* v_pool, int out_dtype, const int32_t* positions,
                                     const int32_t* token_req, const int32_t* block_table, int table_width, int T, int Hq,
                                     int Hkv, int dim, int vdim, const float* q_w, const float* k_w, float eps,
                                     const float* inv_freq, int interleaved, int page_size, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (dim % 2 || dim > QK_MAX_DIM) return gb::fail(GB_UNSUPPORTED, "qk_norm_rope_append: head width %d (even, at most %d)", dim, QK_MAX_DIM);
  if (Hkv > 0 && (!k_pool || !v_pool || !block_table || page_size < 1))
    return gb::fail(GB_BAD_ARGUMENT, "qk_norm_rope_append: kv heads given without a cache to store them in");
  const int heads = Hq + Hkv;
  const int block = heads >= 8 ? 256 : (heads >= 4 ? 128 : 64);
  return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
    return gb::check_pdl_launch(
        gb::launch_pdl(qk_norm_rope_append_kernel<OT>, dim3(T), dim3(block), 0, stream, dim3(1, 1, 1), src, row_stride, q_col,
                       k_col, v_col, (OT*)q_out, (OT*)k_pool, (OT*)v_pool, positions, token_req, block_table, table_width, Hq,
                       Hkv, dim, vdim, q_w, k_w, eps, inv_freq, interleaved, page_size),
        "qk_norm_rope_append");
  });
}

GB_EXPORT int gb_gate_mul(void* x, int x_dtype, const float* gate, int gate_stride, int T, int n, int kind,
                          cudaStream_t stream) {
  if (T <= 0 || n <= 0) return GB_OK;
  if (kind != ACT_SIGMOID && kind != ACT_SILU) return gb::fail(GB_BAD_ARGUMENT, "gate_mul: kind %d", kind);
  if (T > 65535) return gb::fail(GB_UNSUPPORTED, "gate_mul: %d rows (at most 65535 a call)", T);
  const dim3 grid((n + 1023) / 1024, T);
  const bool vec = n % 4 == 0 && gate_stride % 4 == 0 && aligned16(x) && aligned16(gate);
  return GB_DISPATCH_DTYPE(x_dtype, XT, [&]() -> int {
    auto kernel = vec ? gate_mul_kernel<XT, true> : gate_mul_kernel<XT, false>;
    return gb::check_pdl_launch(gb::launch_pdl(kernel, grid, dim3(256), 0, stream, dim3(1, 1, 1), (XT*)x, gate, gate_stride, n, kind),
                                "gate_mul");
  });
}

GB_EXPORT int gb_unary_act(const void* z, int z_dtype, int z_stride, void* out, int out_dtype, int out_stride, int T, int n,
                           int kind, cudaStream_t stream) {
  if (T <= 0 || n <= 0) return GB_OK;
  if (kind < ACT_SIGMOID || kind > ACT_TANH) return gb::fail(GB_BAD_ARGUMENT, "unary_act: kind %d", kind);
  if (T > 65535) return gb::fail(GB_UNSUPPORTED, "unary_act: %d rows (at most 65535 a call)", T);
  const dim3 grid((n + 1023) / 1024, T);
  return GB_DISPATCH_DTYPE(z_dtype, IT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      return gb::check_pdl_launch(gb::launch_pdl(unary_act_kernel<IT, OT>, grid, dim3(256), 0, stream, dim3(1, 1, 1), (const IT*)z,
                                                 z_stride, (OT*)out, out_stride, n, kind),
                                  "unary_act");
    });
  });
}

// ys, ws: `branches` pointers each (ws null: y = ys[0] as it is). x null: the merged row goes to `out`.
// rounded (bfloat16 [T, d], optional): the new x rounded, for the sublayer that reads it next.
GB_EXPORT int gb_sublayer_merge(const float* const* ys, const float* const* ws, int branches, float alpha, float branch_eps,
                                const float* gate, int gate_stride, const float* gate_bias, const float* w, float eps,
                                float* x, float* out, void* rounded, int T, int d, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (branches < 1 || branches > MAX_BRANCHES) return gb::fail(GB_UNSUPPORTED, "sublayer_merge: %d branches (1 to %d)", branches, MAX_BRANCHES);
  if (ws == nullptr && branches != 1) return gb::fail(GB_BAD_ARGUMENT, "sublayer_merge: several branches need their weights");
  if ((x == nullptr) == (out == nullptr)) return gb::fail(GB_BAD_ARGUMENT, "sublayer_merge: either x or out");
  if (x != nullptr && w == nullptr) return gb::fail(GB_BAD_ARGUMENT, "sublayer_merge: the norm's weight is missing");
  if (rounded != nullptr && x == nullptr) return gb::fail(GB_BAD_ARGUMENT, "sublayer_merge: a rounded copy is of x");
  const size_t smem = (size_t)((d + 3) / 4 * 4) * sizeof(float);
  if (smem > 48 * 1024) return gb::fail(GB_UNSUPPORTED, "sublayer_merge: rows of %d (at most 12288)", d);
  Branches br = {};
  br.n = branches;
  bool vec = d % 4 == 0 && gate_stride % 4 == 0 && aligned16(gate) && aligned16(gate_bias) && aligned16(w) && aligned16(x) &&
             aligned16(out) && (reinterpret_cast<uintptr_t>(rounded) & 7) == 0;
  for (int b = 0; b < branches; ++b) {
    br.y[b] = ys[b];
    br.w[b] = ws ? ws[b] : nullptr;
    vec = vec && aligned16(ys[b]) && aligned16(br.w[b]);
  }
  const int threads = d >= 1024 ? 256 : 128;
  auto kernel = vec ? sublayer_merge_kernel<true> : sublayer_merge_kernel<false>;
  return gb::check_pdl_launch(gb::launch_pdl(kernel, dim3(T), dim3(threads), smem, stream, dim3(1, 1, 1), br, alpha, branch_eps,
                                             gate, gate_stride, gate_bias, w, eps, x, out, (__nv_bfloat16*)rounded, d),
                              "sublayer_merge");
}
