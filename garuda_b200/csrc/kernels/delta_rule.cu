// The gated delta rule with a decay per key channel: a recurrent mixer whose state per request and
// head is a matrix S [dim, vdim] in 32-bit, with a short causal convolution in front of its
// query, key and value projections. Per token, in this order:
//     S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// with k and q unit vectors per head (q also times dim^-1/2), beta = sigmoid(.), and
// g = exp(-exp(A_h) softplus(a + dt_bias)) per head and key channel.
//
// Kernels, all 32-bit arithmetic:
//   delta_prepare     a block per token: convolution over the step's rows and the request's kept
//                     last inputs, SiLU, unit vectors, decays, beta
//   delta_conv_state  a request's kept last inputs after the step
//   delta_recurrence  the columns of S are independent of one another, so a request's tokens are
//                     walked in order with no exchange between columns: eight threads share a
//                     column (every eighth row each, in registers) and exchange two sums per token
//                     by shuffles; the step's q, k and g rows come through shared memory a few
//                     tokens at a time
//   delta_out         per head: o / rms(o) * weight * sigmoid(gate)
//   delta_decode      all of the above for steps of one token per request, one block per
//                     (request, head)
// A token's result depends on its request's earlier tokens only through the state, which is
// carried bit for bit: cutting a prompt anywhere gives the same numbers.
#include <type_traits>

#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 8;

__device__ __forceinline__ float silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// Input of channel c at `lag` tokens before token t (index j within its request's rows of this step):
// from the step's rows, or from the request's kept inputs [taps - 1, C] (oldest first).
__device__ __forceinline__ float conv_input(const float* __restrict__ proj, int P, int t, int j, int lag, int c,
                                            const float* __restrict__ kept, int C, int taps) {
  if (j - lag >= 0) return proj[(size_t)(t - lag) * P + c];
  if (kept == nullptr) return 0.f;
  return kept[(size_t)(taps - 1 + j - lag) * C + c];
}

// proj [T, P]: columns q (G dim) | k (G dim) | v (H vdim) | beta (H); the first C = 2 G dim + H vdim are
// the convolved channels. second [T, P2]: its first H dim columns are the decay's pre-activation.
// prep [T, W]: q^ (G dim) | k^ (G dim) | v (H vdim) | g (H dim) | beta (H).
template <typename WT>
__global__ void __launch_bounds__(256)
delta_prepare_kernel(const float* __restrict__ proj, int P, const float* __restrict__ second, int P2,
                     const WT* __restrict__ conv_w, int taps, const float* __restrict__ conv_state,
                     long long state_stride, const WT* __restrict__ a_log, const WT* __restrict__ dt_bias,
                     const int32_t* __restrict__ token_req, const int32_t* __restrict__ cu_q,
                     const int32_t* __restrict__ slots, float* __restrict__ prep, int W, int H, int G, int dim,
                     int vdim, int per_head) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  extern __shared__ float act[];        // [C]
  const int t = blockIdx.x;
  const int r = token_req[t];
  const int j = t - cu_q[r];
  const int slot = slots[r];
  const float* kept = slot >= 0 ? conv_state + (size_t)slot * state_stride : nullptr;
  const int C = 2 * G * dim + H * vdim;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.f;
    for (int tap = 0; tap < taps; ++tap)      // the last column weighs the current token
      acc = fmaf(gb::to_float<WT>(conv_w[(size_t)c * taps + tap]), conv_input(proj, P, t, j, taps - 1 - tap, c, kept, C, taps), acc);
    act[c] = silu(acc);
  }
  __syncthreads();
  float* out = prep + (size_t)t * W;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  // unit vectors: 2 G heads of dim channels, a warp each
  for (int hh = warp; hh < 2 * G; hh += warps) {
    const float* v = act + hh * dim;
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) ss = fmaf(v[d], v[d], ss);
    ss = gb::warp_sum(ss);
    float inv = 1.0f / sqrtf(ss + 1e-6f);
    if (hh < G) inv *= 1.0f / sqrtf((float)dim);
    for (int d = lane; d < dim; d += 32) out[hh * dim + d] = v[d] * inv;
  }
  const int off_v = 2 * G * dim, off_g = off_v + H * vdim, off_b = off_g + H * dim;
  for (int c = threadIdx.x; c < H * vdim; c += blockDim.x) out[off_v + c] = act[off_v + c];
  const float* a = second + (size_t)t * P2;
  // per_head: one decay for all key channels of a head (its pre-activation and bias are per head)
  for (int c = threadIdx.x; c < H * dim; c += blockDim.x) {
    const float rate = expf(gb::to_float<WT>(a_log[c / dim]));
    const int j = per_head ? c / dim : c;
    out[off_g + c] = expf(-rate * softplus(a[j] + gb::to_float<WT>(dt_bias[j])));
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) out[off_b + h] = sigmoid(proj[(size_t)t * P + C + h]);
}

// grid (R, ceil(C / 256)): the request's last taps - 1 inputs after this step, oldest first. A
// thread owns a channel and walks its entries in ascending order, reading only entries above
// the one it writes.
__global__ void __launch_bounds__(256)
delta_conv_state_kernel(const float* __restrict__ proj, int P, float* __restrict__ conv_state, long long state_stride,
                        const int32_t* __restrict__ cu_q, const int32_t* __restrict__ slots, int C, int taps) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const int r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int slot = slots[r];
  if (c >= C || slot < 0) return;
  const int t0 = cu_q[r], n = cu_q[r + 1] - t0;
  float* kept = conv_state + (size_t)slot * state_stride;
  const int keep = taps - 1;
  for (int i = 0; i < keep; ++i) {
    const int src = i + n;                  // index in (kept inputs, then the step's rows)
    kept[(size_t)i * C + c] = src < keep ? kept[(size_t)src * C + c] : proj[(size_t)(t0 + src - keep) * P + c];
  }
}

constexpr int CHUNK = 8;
constexpr int SPLIT = 8;        // threads that share a column of S: thread `sub` holds the rows d with d % 8 == sub
constexpr int REC_THREADS = 128, REC_COLS = REC_THREADS / SPLIT;

__device__ __forceinline__ void cp_async_4(float* smem, const float* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem) : "memory");
}

// grid (H, R, ceil(vdim / 16)), 128 threads: 16 columns of S, eight threads a column. Each of the
// eight sums its rows in ascending order and the eight are added as a tree, ((0 + 1) + (2 + 3)) +
// ((4 + 5) + (6 + 7)): the same sums, in the same order, as the eight interleaved partial sums of
// the one-token kernel below. Everything a token needs (q^, k^, g, the block's values, beta)
// comes through shared memory, eight tokens at a time in two buffers: the next eight are on their
// way while these are walked. EXACT: dim == MAXD, no row of a thread is beyond the head's.
template <int MAXD, bool EXACT>
__global__ void __launch_bounds__(REC_THREADS)
delta_recurrence_kernel(const float* __restrict__ prep, int W, const int32_t* __restrict__ cu_q,
                        const int32_t* __restrict__ slots, float* __restrict__ state, long long state_stride, int H,
                        int G, int dim, int vdim, float* __restrict__ out) {
  gb::pdl_wait();
  constexpr int MINE = MAXD / SPLIT;
  extern __shared__ __align__(16) float stage[];      // 2 x [CHUNK][3 SPLIT per + 32 + 4]
  // a thread's rows, rounded up to whole 16-byte pieces, and one piece more: the four slices start
  // in different banks and are read four values at a time
  const int per = ((dim + SPLIT - 1) / SPLIT + 3) / 4 * 4 + 4;
  const int tok_floats = 3 * SPLIT * per + REC_COLS + 4;      // a multiple of four: every slice starts on 16 bytes
  const int h = blockIdx.x, r = blockIdx.y;
  const int sub = threadIdx.x % SPLIT;
  const int col0 = blockIdx.z * REC_COLS, mycol = threadIdx.x / SPLIT, col = col0 + mycol;
  const bool active = col < vdim;
  const int slot = slots[r];
  const int t0 = cu_q[r], t1 = cu_q[r + 1];
  const int kvh = h / (H / G);
  const int off_q = kvh * dim, off_k = G * dim + kvh * dim, off_v = 2 * G * dim + h * vdim + col0;
  const int off_g = 2 * G * dim + H * vdim + h * dim, off_b = off_g - h * dim + H * dim + h;
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
      const float* row = prep + (size_t)(c0 + tt) * W;
      float* to = dst + tt * tok_floats + (d % SPLIT) * per + d / SPLIT;
      cp_async_4(to, row + off_q + d);
      cp_async_4(to + SPLIT * per, row + off_k + d);
      cp_async_4(to + 2 * SPLIT * per, row + off_g + d);
    }
    for (int i = threadIdx.x; i < n * (ncols + 1); i += REC_THREADS) {
      const int tt = i / (ncols + 1), c = i % (ncols + 1);
      const float* row = prep + (size_t)(c0 + tt) * W;
      float* to = dst + tt * tok_floats + 3 * SPLIT * per;
      if (c < ncols) cp_async_4(to + c, row + off_v + c);
      else cp_async_4(to + REC_COLS, row + off_b);
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
      const float* sq = tok + sub * per;
      const float* sk = sq + SPLIT * per;
      const float* sg = sk + SPLIT * per;
      const float v = active ? tok[3 * SPLIT * per + mycol] : 0.f;
      const float beta = tok[3 * SPLIT * per + REC_COLS];
      float acc = 0.f;
      float kk[MINE];
#pragma unroll
      for (int i4 = 0; i4 < MINE; i4 += 4) {
        if (!EXACT && i4 * SPLIT >= dim) break;         // pieces beyond the head's rows are not in shared memory
        const float4 g4 = *reinterpret_cast<const float4*>(sg + i4);
        const float4 k4 = *reinterpret_cast<const float4*>(sk + i4);
        const float gg[4] = {g4.x, g4.y, g4.z, g4.w};
        kk[i4] = k4.x, kk[i4 + 1] = k4.y, kk[i4 + 2] = k4.z, kk[i4 + 3] = k4.w;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (EXACT || (i4 + j) * SPLIT + sub < dim) {
            S[i4 + j] *= gg[j];
            acc = fmaf(S[i4 + j], kk[i4 + j], acc);
          }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      const float u = beta * (v - acc);
      float o = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < MINE; i4 += 4) {
        if (!EXACT && i4 * SPLIT >= dim) break;
        const float4 q4 = *reinterpret_cast<const float4*>(sq + i4);
        const float qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (EXACT || (i4 + j) * SPLIT + sub < dim) {
            S[i4 + j] = fmaf(kk[i4 + j], u, S[i4 + j]);
            o = fmaf(S[i4 + j], qq[j], o);
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

// A block per token, a warp per head in turn: out[t][h] = o / sqrt(mean(o^2) + eps) * w * act(gate), act =
// sigmoid or SiLU; w [vdim] shared by the heads or [H vdim]. gate: columns gate_off .. of `second`.
template <typename WT, typename OT>
__global__ void __launch_bounds__(128)
delta_out_kernel(const float* __restrict__ o, const float* __restrict__ second, int P2, int gate_off,
                 const WT* __restrict__ w, float eps, OT* __restrict__ out, int H, int vdim, int silu_gate,
                 int w_per_head) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int h = warp; h < H; h += warps) {
    const float* row = o + ((size_t)t * H + h) * vdim;
    const float* gate = second + (size_t)t * P2 + gate_off + h * vdim;
    float ss = 0.f;
    for (int c = lane; c < vdim; c += 32) ss = fmaf(row[c], row[c], ss);
    const float scale = 1.0f / sqrtf(gb::warp_sum(ss) / (float)vdim + eps);
    const WT* wh = w_per_head ? w + (size_t)h * vdim : w;
    for (int c = lane; c < vdim; c += 32)
      out[((size_t)t * H + h) * vdim + c] =
          gb::from_float<OT>((row[c] * scale) * gb::to_float<WT>(wh[c]) * (silu_gate ? silu(gate[c]) : sigmoid(gate[c])));
  }
}

// A step of one token per request: grid (H, R), vdim threads (a column of S each, rounded up to a
// warp). Every block convolves the channels of its own head (its key/value head's q and k, its v),
// so nothing is exchanged between blocks; block h == 0 .. G - 1 also writes nothing extra: the kept
// inputs are shifted by a kernel behind this one. The state column lives in registers for the one
// token: read, decayed, updated, written.
template <int MAXD, typename WT, typename OT>
__global__ void __launch_bounds__(256)
delta_decode_kernel(const float* __restrict__ proj, int P, const float* __restrict__ second, int P2,
                    const WT* __restrict__ conv_w, int taps, const float* __restrict__ conv_state, long long conv_stride,
                    const WT* __restrict__ a_log, const WT* __restrict__ dt_bias, const WT* __restrict__ norm_w, float eps,
                    const int32_t* __restrict__ slots, float* __restrict__ state, long long state_stride, int H, int G,
                    int dim, int vdim, OT* __restrict__ out, int per_head, int gate_off, int silu_gate) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  extern __shared__ float sm[];          // q^[dim], k^[dim], g[dim], scratch[32], o[vdim]
  float* sq = sm;
  float* sk = sm + dim;
  float* sg = sm + 2 * dim;
  float* scratch = sm + 3 * dim;
  const int h = blockIdx.x, t = blockIdx.y;         // one token per request: row t is request t
  const int slot = slots[t];
  const int kvh = h / (H / G);
  const int C = 2 * G * dim + H * vdim;
  const float* kept = slot >= 0 ? conv_state + (size_t)slot * conv_stride : nullptr;
  auto conv = [&](int c) {
    float acc = 0.f;
    for (int tap = 0; tap < taps; ++tap)
      acc = fmaf(gb::to_float<WT>(conv_w[(size_t)c * taps + tap]), conv_input(proj, P, t, 0, taps - 1 - tap, c, kept, C, taps), acc);
    return silu(acc);
  };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    sq[d] = conv(kvh * dim + d);
    sk[d] = conv(G * dim + kvh * dim + d);
    const int c = per_head ? h : h * dim + d;
    sg[d] = expf(-expf(gb::to_float<WT>(a_log[h])) * softplus(second[(size_t)t * P2 + c] + gb::to_float<WT>(dt_bias[c])));
  }
  __syncthreads();
  // unit vectors: warp 0 the query, warp 1 (or 0 again) the key
  for (int which = warp; which < 2; which += warps) {
    float* v = which == 0 ? sq : sk;
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) ss = fmaf(v[d], v[d], ss);
    ss = gb::warp_sum(ss);
    float inv = 1.0f / sqrtf(ss + 1e-6f);
    if (which == 0) inv *= 1.0f / sqrtf((float)dim);
    __syncwarp();
    for (int d = lane; d < dim; d += 32) v[d] *= inv;
  }
  __syncthreads();
  const int col = threadIdx.x;
  const bool active = col < vdim;
  float o_val = 0.f;
  if (active) {
    const float v = conv(2 * G * dim + h * vdim + col);
    const float beta = sigmoid(proj[(size_t)t * P + C + h]);
    float* S_g = slot >= 0 ? state + (size_t)slot * state_stride + (size_t)h * dim * vdim + col : nullptr;
    float S[MAXD];
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int d = 0; d < MAXD; ++d)
      if (d < dim) {
        S[d] = (S_g != nullptr ? S_g[(size_t)d * vdim] : 0.f) * sg[d];
        acc[d & 7] = fmaf(S[d], sk[d], acc[d & 7]);
      }
    // the tree the kernel for longer steps adds its eight threads' sums by
    const float u = beta * (v - (((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]))));
    float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int d = 0; d < MAXD; ++d)
      if (d < dim) {
        S[d] = fmaf(sk[d], u, S[d]);
        o[d & 7] = fmaf(S[d], sq[d], o[d & 7]);
        if (S_g != nullptr) S_g[(size_t)d * vdim] = S[d];
      }
    o_val = ((o[0] + o[1]) + (o[2] + o[3])) + ((o[4] + o[5]) + (o[6] + o[7]));
  }
  // the head's RMS over vdim, the weight and the output gate; the sum of squares in the order the
  // kernel for longer steps takes it (a lane's channels in ascending order, then the warp's tree),
  // so that a token's result is the same bits whichever kernel ran it
  float* so = scratch + 32;            // [vdim]
  if (active) so[col] = o_val;
  __syncthreads();
  float ss = 0.f;
  for (int c = lane; c < vdim; c += 32) ss = fmaf(so[c], so[c], ss);
  const float scale = 1.0f / sqrtf(gb::warp_sum(ss) / (float)vdim + eps);
  if (active) {
    const float gate = second[(size_t)t * P2 + gate_off + h * vdim + col];
    out[((size_t)t * H + h) * vdim + col] =
        gb::from_float<OT>((o_val * scale) * gb::to_float<WT>(norm_w[col]) * (silu_gate ? silu(gate) : sigmoid(gate)));
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

int check_sizes(const char* what, int H, int G, int dim, int vdim, int taps) {
  if (H < 1 || G < 1 || H % G) return gb::fail(GB_BAD_ARGUMENT, "%s: %d heads for %d key heads", what, H, G);
  if (dim < 1 || vdim < 1) return gb::fail(GB_BAD_ARGUMENT, "%s: head sizes %d and %d", what, dim, vdim);
  if (taps < 1 || taps > MAX_TAPS) return gb::fail(GB_UNSUPPORTED, "%s: %d taps (1 to %d)", what, taps, MAX_TAPS);
  return GB_OK;
}

}  // namespace

// state_stride, conv_stride: floats between two slots' states.
GB_EXPORT int gb_delta_prepare(const float* proj, int P, const float* second, int P2, const void* conv_w, int w_dtype,
                               int taps, const float* conv_state, long long conv_stride, const void* a_log,
                               const void* dt_bias, const int32_t* token_req, const int32_t* cu_q, const int32_t* slots,
                               float* prep, int W, int T, int H, int G, int dim, int vdim, int per_head,
                               cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  int rc = check_sizes("delta_prepare", H, G, dim, vdim, taps);
  if (rc != GB_OK) return rc;
  const int C = 2 * G * dim + H * vdim;
  if (P < C + H || P2 < (per_head ? H : H * dim) || W != C + H * dim + H)
    return gb::fail(GB_BAD_ARGUMENT, "delta_prepare: row widths");
  const size_t smem = (size_t)C * sizeof(float);
  constexpr size_t kMostSmem = 224 * 1024;      // what a block may ask for on this GPU, less some for the driver
  if (smem > kMostSmem) return gb::fail(GB_UNSUPPORTED, "delta_prepare: %d convolved channels (at most %d)", C, (int)(kMostSmem / 4));
  return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
    if (smem > 48 * 1024) {                      // beyond the default limit a kernel has to ask once
      static size_t granted = 0;                 // per weight type: this lambda is instantiated for each
      if (smem > granted) {
        const cudaError_t e = cudaFuncSetAttribute(delta_prepare_kernel<WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMostSmem);
        if (e != cudaSuccess) return gb::fail(GB_CUDA_ERROR, "delta_prepare: %s", cudaGetErrorString(e));
        granted = kMostSmem;
      }
    }
    return gb::check_pdl_launch(
        gb::launch_pdl(delta_prepare_kernel<WT>, dim3(T), dim3(256), smem, stream, dim3(1, 1, 1), proj, P, second, P2,
                       (const WT*)conv_w, taps, conv_state, conv_stride, (const WT*)a_log, (const WT*)dt_bias, token_req,
                       cu_q, slots, prep, W, H, G, dim, vdim, per_head),
        "delta_prepare");
  });
}

GB_EXPORT int gb_delta_conv_state(const float* proj, int P, float* conv_state, long long conv_stride, const int32_t* cu_q,
                                  const int32_t* slots, int R, int C, int taps, cudaStream_t stream) {
  if (R <= 0 || taps <= 1) return GB_OK;
  return gb::check_pdl_launch(gb::launch_pdl(delta_conv_state_kernel, dim3(R, (C + 255) / 256), dim3(256), 0, stream,
                                             dim3(1, 1, 1), proj, P, conv_state, conv_stride, cu_q, slots, C, taps),
                              "delta_conv_state");
}

GB_EXPORT int gb_delta_recurrence(const float* prep, int W, const int32_t* cu_q, const int32_t* slots, float* state,
                                  long long state_stride, int R, int H, int G, int dim, int vdim, float* out,
                                  cudaStream_t stream) {
  if (R <= 0) return GB_OK;
  int rc = check_sizes("delta_recurrence", H, G, dim, vdim, 1);
  if (rc != GB_OK) return rc;
  const int threads = REC_THREADS, cols = REC_COLS;
  const dim3 grid(H, R, (vdim + cols - 1) / cols);
  const int per = ((dim + SPLIT - 1) / SPLIT + 3) / 4 * 4 + 4;
  const size_t smem = (size_t)2 * CHUNK * (3 * SPLIT * per + REC_COLS + 4) * sizeof(float);
  return by_dim(dim, "delta_recurrence", [&](auto maxd) -> int {
    if (smem > 48 * 1024) {     // never with these tile sizes (key widths up to 256 need 34 KB); kept for larger ones
      cudaError_t e1 = cudaFuncSetAttribute(delta_recurrence_kernel<decltype(maxd)::value, true>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      cudaError_t e2 = cudaFuncSetAttribute(delta_recurrence_kernel<decltype(maxd)::value, false>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e1 != cudaSuccess || e2 != cudaSuccess) return gb::fail(GB_CUDA_ERROR, "delta_recurrence: shared memory");
    }
    constexpr int MAXD = decltype(maxd)::value;
    auto kernel = dim == MAXD ? delta_recurrence_kernel<MAXD, true> : delta_recurrence_kernel<MAXD, false>;
    return gb::check_pdl_launch(gb::launch_after(kernel, grid, dim3(threads), smem, stream, dim3(1, 1, 1), prep, W, cu_q,
                                               slots, state, state_stride, H, G, dim, vdim, out),
                                "delta_recurrence");
  });
}

GB_EXPORT int gb_delta_out(const float* o, const float* second, int P2, int gate_off, const void* w, int w_dtype,
                           float eps, void* out, int out_dtype, int T, int H, int vdim, int silu_gate, int w_per_head,
                           cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      return gb::check_pdl_launch(gb::launch_pdl(delta_out_kernel<WT, OT>, dim3(T), dim3(128), 0, stream, dim3(1, 1, 1), o,
                                                 second, P2, gate_off, (const WT*)w, eps, (OT*)out, H, vdim, silu_gate,
                                                 w_per_head),
                                  "delta_out");
    });
  });
}

// One token per request (row t of the batch is request t). Takes vdim <= 256.
GB_EXPORT int gb_delta_decode(const float* proj, int P, const float* second, int P2, const void* conv_w, int w_dtype,
                              int taps, const float* conv_state, long long conv_stride, const void* a_log,
                              const void* dt_bias, const void* norm_w, float eps, const int32_t* slots, float* state,
                              long long state_stride, int R, int H, int G, int dim, int vdim, void* out, int out_dtype,
                              int per_head, int gate_off, int silu_gate, cudaStream_t stream) {
  if (R <= 0) return GB_OK;
  int rc = check_sizes("delta_decode", H, G, dim, vdim, taps);
  if (rc != GB_OK) return rc;
  if (vdim > 256) return gb::fail(GB_UNSUPPORTED, "delta_decode: %d value channels per head (at most 256)", vdim);
  const int threads = (vdim + 31) / 32 * 32;
  const size_t smem = (size_t)(3 * dim + 32 + vdim) * sizeof(float);
  return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      return by_dim(dim, "delta_decode", [&](auto maxd) -> int {
        return gb::check_pdl_launch(
            gb::launch_pdl(delta_decode_kernel<decltype(maxd)::value, WT, OT>, dim3(H, R), dim3(threads), smem, stream,
                           dim3(1, 1, 1), proj, P, second, P2, (const WT*)conv_w, taps, conv_state, conv_stride,
                           (const WT*)a_log, (const WT*)dt_bias, (const WT*)norm_w, eps, slots, state, state_stride, H, G,
                           dim, vdim, (OT*)out, per_head, gate_off, silu_gate),
            "delta_decode");
      });
    });
  });
}
