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

template <typename XT>
__global__ void gate_mul_kernel(XT* __restrict__ x, const float* __restrict__ gate, int gate_stride, long long total,
                                int n, int kind) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / n;
    const int c = (int)(i % n);
    x[i] = gb::from_float<XT>(gb::to_float<XT>(x[i]) * act(gate[t * gate_stride + c], kind));
  }
}

template <typename IT, typename OT>
__global__ void unary_act_kernel(const IT* __restrict__ z, int z_stride, OT* __restrict__ out, int out_stride,
                                 long long total, int n, int kind) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / n;
    const int c = (int)(i % n);
    out[t * out_stride + c] = gb::from_float<OT>(act(gb::to_float<IT>(z[t * z_stride + c]), kind));
  }
}

constexpr int MAX_BRANCHES = 4;
struct Branches {
  const float* y[MAX_BRANCHES];
  const float* w[MAX_BRANCHES];
  int n;
};

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = gb::warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  __syncthreads();                  // `red` may still be read from the call before
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int i = 0; i < warps; ++i) total += red[i];      // every thread adds in the same order
  return total;
}

// One block per token; the row lives in shared memory between the passes.
__global__ void __launch_bounds__(256)
sublayer_merge_kernel(Branches br, float alpha, float branch_eps, const float* __restrict__ gate, int gate_stride,
                      const float* __restrict__ gate_bias, const float* __restrict__ w, float eps, float* __restrict__ x,
                      float* __restrict__ out, __nv_bfloat16* __restrict__ rounded, int d) {
  extern __shared__ float rowbuf[];       // [d]
  __shared__ float red[8];
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const size_t t = blockIdx.x;
  if (br.w[0] != nullptr) {
    for (int c = threadIdx.x; c < d; c += blockDim.x) rowbuf[c] = 0.f;
    for (int b = 0; b < br.n; ++b) {
      const float* y = br.y[b] + t * d;
      float ss = 0.f;
      for (int c = threadIdx.x; c < d; c += blockDim.x) ss = fmaf(y[c], y[c], ss);
      const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + branch_eps);
      for (int c = threadIdx.x; c < d; c += blockDim.x) rowbuf[c] += (y[c] * inv) * br.w[b][c];
    }
    for (int c = threadIdx.x; c < d; c += blockDim.x) rowbuf[c] *= alpha;
  } else {
    const float* y = br.y[0] + t * d;
    for (int c = threadIdx.x; c < d; c += blockDim.x) rowbuf[c] = y[c];
  }
  if (gate != nullptr) {
    const float* g = gate + t * gate_stride;
    for (int c = threadIdx.x; c < d; c += blockDim.x)
      rowbuf[c] *= sigmoidf_(g[c] + (gate_bias ? gate_bias[c] : 0.f));
  }
  if (x == nullptr) {
    for (int c = threadIdx.x; c < d; c += blockDim.x) out[t * d + c] = rowbuf[c];
    return;
  }
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) ss = fmaf(rowbuf[c], rowbuf[c], ss);
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float v = x[t * d + c] + (rowbuf[c] * inv) * w[c];
    x[t * d + c] = v;
    if (rounded != nullptr) rounded[t * d + c] = __float2bfloat16_rn(v);
  }
}

int grid_for(long long total, int block) {
  long long g = (total + block - 1) / block;
  return (int)(g > 148 * 32 ? 148 * 32 : (g < 1 ? 1 : g));
}

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
  const long long total = (long long)T * n;
  return GB_DISPATCH_DTYPE(x_dtype, XT, [&]() -> int {
    return gb::check_pdl_launch(gb::launch_pdl(gate_mul_kernel<XT>, dim3(grid_for(total, 256)), dim3(256), 0, stream,
                                               dim3(1, 1, 1), (XT*)x, gate, gate_stride, total, n, kind),
                                "gate_mul");
  });
}

GB_EXPORT int gb_unary_act(const void* z, int z_dtype, int z_stride, void* out, int out_dtype, int out_stride, int T, int n,
                           int kind, cudaStream_t stream) {
  if (T <= 0 || n <= 0) return GB_OK;
  if (kind < ACT_SIGMOID || kind > ACT_TANH) return gb::fail(GB_BAD_ARGUMENT, "unary_act: kind %d", kind);
  const long long total = (long long)T * n;
  return GB_DISPATCH_DTYPE(z_dtype, IT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      return gb::check_pdl_launch(gb::launch_pdl(unary_act_kernel<IT, OT>, dim3(grid_for(total, 256)), dim3(256), 0, stream,
                                                 dim3(1, 1, 1), (const IT*)z, z_stride, (OT*)out, out_stride, total, n, kind),
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
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 48 * 1024) return gb::fail(GB_UNSUPPORTED, "sublayer_merge: rows of %d (at most 12288)", d);
  Branches br = {};
  br.n = branches;
  for (int b = 0; b < branches; ++b) {
    br.y[b] = ys[b];
    br.w[b] = ws ? ws[b] : nullptr;
  }
  return gb::check_pdl_launch(gb::launch_pdl(sublayer_merge_kernel, dim3(T), dim3(256), smem, stream, dim3(1, 1, 1), br, alpha,
                                             branch_eps, gate, gate_stride, gate_bias, w, eps, x, out, (__nv_bfloat16*)rounded, d),
                              "sublayer_merge");
}
