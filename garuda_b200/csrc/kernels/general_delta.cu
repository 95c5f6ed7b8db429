// The generalized delta rule: a recurrent mixer whose state per request and head is a matrix
// S [dim, vdim] in 32-bit. Per token, with r, k, v the projected rows, w a decay and a a removal
// rate per head and key channel, and u = k / sqrt(sum k^2 + 1e-6) the head's unit key:
//     S <- diag(w) S - (a * u) (u^T S) + k v^T      (both terms read the old S)
//     o  = S^T r
//     w  = exp(-c sigmoid(z + w0)),   a = sigmoid(y + a0)
// with z the decay's pre-activation (a low-rank pair of products), y the removal's, c a constant.
//
// Column c of S, u^T S at c and o_c involve no other column, so a request's tokens are walked in
// order with no exchange between columns. Kernels, all 32-bit arithmetic:
//   gdelta_prepare      a block per token: decays, removal rates, unit keys
//   gdelta_recurrence   eight threads share a column (every eighth row each, in registers) and
//                       exchange two sums per token by shuffles; a token's r, u, w, a*u, k come
//                       through shared memory, eight (or four) tokens at a time in two buffers
//   gdelta_decode       all of it, with the read-out's norm, weight and gate, for steps of one
//                       token per request: a block per (request, head)
// The read-out's norm for longer steps is delta_out (delta_rule.cu). A token's result depends on
// its request's earlier tokens only through the state, which is carried bit for bit.
#include <type_traits>

#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// proj [T, P]: columns r | k | v | removal logits | ...; each block H dim wide (v: H vdim).
// zdec [T, PZ]: the decay's pre-activation, H dim wide.
// prep [T, W]: r | u | w | a*u | k  (H dim each) | v (H vdim).
__global__ void __launch_bounds__(256)
gdelta_prepare_kernel(const float* __restrict__ proj, int P, int col_r, int col_k, int col_v, int col_a,
                      const float* __restrict__ zdec, int PZ, const float* __restrict__ w0, const float* __restrict__ a0,
                      float decay_scale, float* __restrict__ prep, int W, int H, int dim, int vdim) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const size_t t = blockIdx.x;
  const float* row = proj + t * P;
  float* out = prep + t * W;
  const int HD = H * dim;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int h = warp; h < H; h += warps) {
    const float* k = row + col_k + h * dim;
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) ss = fmaf(k[d], k[d], ss);
    const float inv = 1.0f / sqrtf(gb::warp_sum(ss) + 1e-6f);
    for (int d = lane; d < dim; d += 32) {
      const int c = h * dim + d;
      const float u = k[d] * inv;
      out[c] = row[col_r + c];
      out[HD + c] = u;
      out[2 * HD + c] = expf(-decay_scale * sigmoid(zdec[t * PZ + c] + w0[c]));
      out[3 * HD + c] = sigmoid(row[col_a + c] + a0[c]) * u;
      out[4 * HD + c] = k[d];
    }
  }
  for (int c = threadIdx.x; c < H * vdim; c += blockDim.x) out[5 * HD + c] = row[col_v + c];
}

constexpr int SPLIT = 8;        // threads that share a column of S: thread `sub` holds the rows d with d % 8 == sub
constexpr int REC_THREADS = 128, REC_COLS = REC_THREADS / SPLIT;
constexpr int VECS = 5;         // r, u, w, a*u, k

__device__ __forceinline__ void cp_async_4(float* smem, const float* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem) : "memory");
}

// grid (H, R, ceil(vdim / 16)), 128 threads: 16 columns of S, eight threads a column. Each of the
// eight sums its rows in ascending order and the eight are added as a tree, ((0 + 1) + (2 + 3)) +
// ((4 + 5) + (6 + 7)): the same sums, in the same order, as the eight interleaved partial sums of
// the one-token kernel below. EXACT: dim == MAXD, no row of a thread is beyond the head's.
template <int MAXD, bool EXACT, int CHUNK>
__global__ void __launch_bounds__(REC_THREADS)
gdelta_recurrence_kernel(const float* __restrict__ prep, int W, const int32_t* __restrict__ cu_q,
                         const int32_t* __restrict__ slots, float* __restrict__ state, long long state_stride, int H,
                         int dim, int vdim, float* __restrict__ out) {
  gb::pdl_wait();
  constexpr int MINE = MAXD / SPLIT;
  extern __shared__ __align__(16) float stage[];      // 2 x [CHUNK][VECS SPLIT per + 16 + 4]
  const int per = ((dim + SPLIT - 1) / SPLIT + 3) / 4 * 4 + 4;
  const int tok_floats = VECS * SPLIT * per + REC_COLS + 4;
  const int h = blockIdx.x, r = blockIdx.y;
  const int sub = threadIdx.x % SPLIT;
  const int col0 = blockIdx.z * REC_COLS, mycol = threadIdx.x / SPLIT, col = col0 + mycol;
  const bool active = col < vdim;
  const int slot = slots[r];
  const int t0 = cu_q[r], t1 = cu_q[r + 1];
  const int HD = H * dim;
  const int off_v = VECS * HD + h * vdim + col0;
  const int ncols = min(REC_COLS, vdim - col0);
  float* S_g = (slot >= 0 && active) ? state + (size_t)slot * state_stride + (size_t)h * dim * vdim + col : nullptr;
  float S[MINE];
#pragma unroll
  for (int i = 0; i < MINE; ++i) {
    const int d = i * SPLIT + sub;
    S[i] = (d < dim && S_g != nullptr) ? S_g[(size_t)d * vdim] : 0.f;
  }
  auto fetch = [&](int c0, int buf) {
    const int n = min(CHUNK, t1 - c0);
    float* dst = stage + (size_t)buf * CHUNK * tok_floats;
    for (int i = threadIdx.x; i < n * dim; i += REC_THREADS) {
      const int tt = i / dim, d = i % dim;
      const float* row = prep + (size_t)(c0 + tt) * W + h * dim + d;
      float* to = dst + tt * tok_floats + (d % SPLIT) * per + d / SPLIT;
#pragma unroll
      for (int v = 0; v < VECS; ++v) cp_async_4(to + v * SPLIT * per, row + v * HD);
    }
    for (int i = threadIdx.x; i < n * ncols; i += REC_THREADS) {
      const int tt = i / ncols, c = i % ncols;
      cp_async_4(dst + tt * tok_floats + VECS * SPLIT * per + c, prep + (size_t)(c0 + tt) * W + off_v + c);
    }
  };
  if (t0 < t1) fetch(t0, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");
  int buf = 0;
  for (int c0 = t0; c0 < t1; c0 += CHUNK, buf ^= 1) {
    const int n = min(CHUNK, t1 - c0);
    if (c0 + CHUNK < t1) fetch(c0 + CHUNK, buf ^ 1);       // that buffer was read two rounds ago, behind a barrier
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    const float* cur = stage + (size_t)buf * CHUNK * tok_floats;
    // unrolled: a token's read-out (its sum and shuffles) is off the path to the next token's state and overlaps it
#pragma unroll 4
    for (int tt = 0; tt < n; ++tt) {
      const float* tok = cur + tt * tok_floats;
      const float* sr = tok + sub * per;
      const float* su = sr + SPLIT * per;
      const float* sw = su + SPLIT * per;
      const float* sa = sw + SPLIT * per;
      const float* sk = sa + SPLIT * per;
      const float v = active ? tok[VECS * SPLIT * per + mycol] : 0.f;
      float acc = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < MINE; i4 += 4) {
        if (!EXACT && i4 * SPLIT >= dim) break;         // pieces beyond the head's rows are not in shared memory
        const float4 u4 = *reinterpret_cast<const float4*>(su + i4);
        const float uu[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (EXACT || (i4 + j) * SPLIT + sub < dim) acc = fmaf(S[i4 + j], uu[j], acc);
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      float o = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < MINE; i4 += 4) {
        if (!EXACT && i4 * SPLIT >= dim) break;
        const float4 w4 = *reinterpret_cast<const float4*>(sw + i4);
        const float4 a4 = *reinterpret_cast<const float4*>(sa + i4);
        const float4 k4 = *reinterpret_cast<const float4*>(sk + i4);
        const float4 r4 = *reinterpret_cast<const float4*>(sr + i4);
        const float ww[4] = {w4.x, w4.y, w4.z, w4.w}, aa[4] = {a4.x, a4.y, a4.z, a4.w};
        const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, rr[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (EXACT || (i4 + j) * SPLIT + sub < dim) {
            S[i4 + j] = fmaf(kk[j], v, fmaf(-aa[j], acc, ww[j] * S[i4 + j]));
            o = fmaf(S[i4 + j], rr[j], o);
          }
      }
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      o += __shfl_xor_sync(0xffffffffu, o, 4);
      if (active && sub == 0) out[(size_t)(c0 + tt) * H * vdim + h * vdim + col] = o;
    }
    __syncthreads();
  }
  // only now may the next kernel in the stream start: its blocks would wait beside these for the whole walk
  gb::pdl_launch_dependents();
  if (S_g != nullptr) {
#pragma unroll
    for (int i = 0; i < MINE; ++i) {
      const int d = i * SPLIT + sub;
      if (d < dim) S_g[(size_t)d * vdim] = S[i];
    }
  }
}

// A step of one token per request: grid (H, R), vdim threads (a column of S each, rounded up to a
// warp). The state column lives in registers for the one token: read, updated, written. The sums
// are taken as the kernel for longer steps takes them, so a token's result is the same bits
// whichever kernel ran it.
template <int MAXD, typename OT>
__global__ void __launch_bounds__(256)
gdelta_decode_kernel(const float* __restrict__ proj, int P, int col_r, int col_k, int col_v, int col_a, int col_g,
                     const float* __restrict__ zdec, int PZ, const float* __restrict__ w0, const float* __restrict__ a0,
                     float decay_scale, const float* __restrict__ norm_w, float eps, const int32_t* __restrict__ slots,
                     float* __restrict__ state, long long state_stride, int H, int dim, int vdim, OT* __restrict__ out) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  extern __shared__ float sm[];          // r, u, w, a*u, k [dim each], o [vdim]
  float* sr = sm;
  float* su = sm + dim;
  float* sw = sm + 2 * dim;
  float* sa = sm + 3 * dim;
  float* sk = sm + 4 * dim;
  float* so = sm + 5 * dim;
  const int h = blockIdx.x;
  const size_t t = blockIdx.y;            // one token per request: row t is request t
  const int slot = slots[t];
  const float* row = proj + t * P;
  const int lane = threadIdx.x & 31;
  // the unit key: every warp takes the sum itself (a lane's channels in ascending order, then the tree)
  float ss = 0.f;
  for (int d = lane; d < dim; d += 32) {
    const float k = row[col_k + h * dim + d];
    ss = fmaf(k, k, ss);
  }
  const float inv = 1.0f / sqrtf(gb::warp_sum(ss) + 1e-6f);
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    const int c = h * dim + d;
    const float k = row[col_k + c], u = k * inv;
    sr[d] = row[col_r + c];
    su[d] = u;
    sw[d] = expf(-decay_scale * sigmoid(zdec[t * PZ + c] + w0[c]));
    sa[d] = sigmoid(row[col_a + c] + a0[c]) * u;
    sk[d] = k;
  }
  __syncthreads();
  const int col = threadIdx.x;
  const bool active = col < vdim;
  float o_val = 0.f;
  if (active) {
    const float v = row[col_v + h * vdim + col];
    float* S_g = slot >= 0 ? state + (size_t)slot * state_stride + (size_t)h * dim * vdim + col : nullptr;
    float S[MAXD];
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int d = 0; d < MAXD; ++d)
      if (d < dim) {
        S[d] = S_g != nullptr ? S_g[(size_t)d * vdim] : 0.f;
        acc[d & 7] = fmaf(S[d], su[d], acc[d & 7]);
      }
    const float dot = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
    float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int d = 0; d < MAXD; ++d)
      if (d < dim) {
        S[d] = fmaf(sk[d], v, fmaf(-sa[d], dot, sw[d] * S[d]));
        o[d & 7] = fmaf(S[d], sr[d], o[d & 7]);
        if (S_g != nullptr) S_g[(size_t)d * vdim] = S[d];
      }
    o_val = ((o[0] + o[1]) + (o[2] + o[3])) + ((o[4] + o[5]) + (o[6] + o[7]));
    so[col] = o_val;
  }
  __syncthreads();
  float sq = 0.f;
  for (int c = lane; c < vdim; c += 32) sq = fmaf(so[c], so[c], sq);
  const float scale = 1.0f / sqrtf(gb::warp_sum(sq) / (float)vdim + eps);
  if (active) {
    const float gate = row[col_g + h * vdim + col];
    out[(t * H + h) * vdim + col] = gb::from_float<OT>((o_val * scale) * norm_w[h * vdim + col] * sigmoid(gate));
  }
}

template <typename F>
int by_dim(int dim, const char* what, F&& f) {
  if (dim <= 32) return f(std::integral_constant<int, 32>());
  if (dim <= 64) return f(std::integral_constant<int, 64>());
  if (dim <= 128) return f(std::integral_constant<int, 128>());
  if (dim <= 256) return f(std::integral_constant<int, 256>());
  return gb::fail(GB_UNSUPPORTED, "%s: %d key channels per head (at most 256)", what, dim);
}

}  // namespace

GB_EXPORT int gb_gdelta_prepare(const float* proj, int P, int col_r, int col_k, int col_v, int col_a, const float* zdec,
                                int PZ, const float* w0, const float* a0, float decay_scale, float* prep, int W, int T, int H,
                                int dim, int vdim, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (H < 1 || dim < 1 || vdim < 1) return gb::fail(GB_BAD_ARGUMENT, "gdelta_prepare: sizes");
  if (W != 5 * H * dim + H * vdim || PZ < H * dim) return gb::fail(GB_BAD_ARGUMENT, "gdelta_prepare: row widths");
  return gb::check_pdl_launch(gb::launch_pdl(gdelta_prepare_kernel, dim3(T), dim3(256), 0, stream, dim3(1, 1, 1), proj, P, col_r,
                                             col_k, col_v, col_a, zdec, PZ, w0, a0, decay_scale, prep, W, H, dim, vdim),
                              "gdelta_prepare");
}

GB_EXPORT int gb_gdelta_recurrence(const float* prep, int W, const int32_t* cu_q, const int32_t* slots, float* state,
                                   long long state_stride, int R, int H, int dim, int vdim, float* out, cudaStream_t stream) {
  if (R <= 0) return GB_OK;
  if (H < 1 || dim < 1 || vdim < 1) return gb::fail(GB_BAD_ARGUMENT, "gdelta_recurrence: sizes");
  const dim3 grid(H, R, (vdim + REC_COLS - 1) / REC_COLS);
  const int per = ((dim + SPLIT - 1) / SPLIT + 3) / 4 * 4 + 4;
  const size_t tok = (size_t)(VECS * SPLIT * per + REC_COLS + 4) * sizeof(float);
  // eight tokens at a time where two buffers of them fit in 48 KB (up to 64 key channels), else four (47 KB at 256)
  const bool eight = 2 * 8 * tok <= 48 * 1024;
  const size_t smem = 2 * (eight ? 8 : 4) * tok;
  if (smem > 48 * 1024) return gb::fail(GB_UNSUPPORTED, "gdelta_recurrence: %d key channels per head", dim);
  return by_dim(dim, "gdelta_recurrence", [&](auto maxd) -> int {
    constexpr int MAXD = decltype(maxd)::value;
    auto kernel = eight ? (dim == MAXD ? gdelta_recurrence_kernel<MAXD, true, 8> : gdelta_recurrence_kernel<MAXD, false, 8>)
                        : (dim == MAXD ? gdelta_recurrence_kernel<MAXD, true, 4> : gdelta_recurrence_kernel<MAXD, false, 4>);
    return gb::check_pdl_launch(gb::launch_after(kernel, grid, dim3(REC_THREADS), smem, stream, dim3(1, 1, 1), prep, W, cu_q, slots,
                                               state, state_stride, H, dim, vdim, out),
                                "gdelta_recurrence");
  });
}

// One token per request (row t of the batch is request t). Takes vdim <= 256.
GB_EXPORT int gb_gdelta_decode(const float* proj, int P, int col_r, int col_k, int col_v, int col_a, int col_g,
                               const float* zdec, int PZ, const float* w0, const float* a0, float decay_scale,
                               const float* norm_w, float eps, const int32_t* slots, float* state, long long state_stride,
                               int R, int H, int dim, int vdim, void* out, int out_dtype, cudaStream_t stream) {
  if (R <= 0) return GB_OK;
  if (H < 1 || dim < 1 || vdim < 1) return gb::fail(GB_BAD_ARGUMENT, "gdelta_decode: sizes");
  if (vdim > 256) return gb::fail(GB_UNSUPPORTED, "gdelta_decode: %d value channels per head (at most 256)", vdim);
  const int threads = (vdim + 31) / 32 * 32;
  const size_t smem = (size_t)(5 * dim + vdim) * sizeof(float);
  return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
    return by_dim(dim, "gdelta_decode", [&](auto maxd) -> int {
      return gb::check_pdl_launch(
          gb::launch_pdl(gdelta_decode_kernel<decltype(maxd)::value, OT>, dim3(H, R), dim3(threads), smem, stream,
                         dim3(1, 1, 1), proj, P, col_r, col_k, col_v, col_a, col_g, zdec, PZ, w0, a0, decay_scale, norm_w, eps,
                         slots, state, state_stride, H, dim, vdim, (OT*)out),
          "gdelta_decode");
    });
  });
}
