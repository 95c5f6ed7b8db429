// minGRU: a recurrence per channel c whose gate and candidate are functions of the current token alone:
//
//   z_t = sigmoid(a_t + bz)          a, u, g: three column ranges of one projected 32-bit row
//   n_t = u_t + bu + 1/2  where u_t + bu >= 0,  sigmoid(u_t + bu)  below
//   S_t = (1 - z_t) S_(t-1) + z_t n_t
//   out_t = S_t * silu(g_t)
//
// S lives in a 32-bit row per request slot and is carried from step to step. Everything is 32-bit
// arithmetic; only `out` is rounded to the compute dtype.
//
// The recurrence S_t = p_t S_(t-1) + b_t is linear in S, so a stretch of tokens acts on what comes in as
// S -> P S + B with P the product of its p and B its result from zero. Steps whose longest request has
// at most SEG tokens (decode among them) run one kernel, a thread per (request, channel) walking the
// tokens. Longer steps cut every request into stretches of SEG tokens: a first kernel takes each
// stretch's (P, B), a second one folds the stretches in front into the incoming state (at most a few
// dozen multiply-adds) and walks its own stretch again, now from the right start. A request's tokens
// are thus worked on by ceil(len / SEG) blocks per 128 channels instead of one.
#include "common.cuh"

namespace {

constexpr int SEG = 64;
constexpr int THREADS = 128;

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

struct Rows {
  const float* proj;
  long long stride;
  int z_col, u_col, g_col;
  const float* bz;
  const float* bu;
};

// p = 1 - z and b = z * candidate of channel c at token t
__device__ __forceinline__ void gates(const Rows& in, long long t, int c, float bz, float bu, float& p, float& b) {
  const float* row = in.proj + t * in.stride;
  const float z = sigmoidf_(row[in.z_col + c] + bz);
  const float u = row[in.u_col + c] + bu;
  const float n = u >= 0.f ? u + 0.5f : sigmoidf_(u);
  p = 1.0f - z;
  b = z * n;
}

constexpr int AHEAD = 8;      // tokens whose rows a thread asks for before it needs the first of them

// Walks tokens [t0, t1) of channel c from S, writing the gated read-out; returns the last S. The
// rows of AHEAD tokens are loaded before the chain of multiply-adds over them runs: what bounds a
// walk is the loads' latency, and nothing in a load depends on S.
template <typename OT>
__device__ __forceinline__ float walk(const Rows& in, int t0, int t1, int c, float bz, float bu, float S, OT* out, int W) {
  int t = t0;
  for (; t + AHEAD <= t1; t += AHEAD) {
    float a[AHEAD], u[AHEAD], g[AHEAD];
#pragma unroll
    for (int k = 0; k < AHEAD; ++k) {
      const float* row = in.proj + (long long)(t + k) * in.stride;
      a[k] = row[in.z_col + c];
      u[k] = row[in.u_col + c];
      g[k] = row[in.g_col + c];
    }
#pragma unroll
    for (int k = 0; k < AHEAD; ++k) {
      const float z = sigmoidf_(a[k] + bz), v = u[k] + bu;
      const float n = v >= 0.f ? v + 0.5f : sigmoidf_(v);
      S = fmaf(1.0f - z, S, z * n);
      out[(size_t)(t + k) * W + c] = gb::from_float<OT>(S * (g[k] * sigmoidf_(g[k])));
    }
  }
  for (; t < t1; ++t) {
    float p, b;
    gates(in, t, c, bz, bu, p, b);
    S = fmaf(p, S, b);
    const float g = in.proj[(long long)t * in.stride + in.g_col + c];
    out[(size_t)t * W + c] = gb::from_float<OT>(S * (g * sigmoidf_(g)));
  }
  return S;
}

// grid (ceil(W / THREADS), requests): the whole of a request's tokens of this step, from its state.
// A row whose slot is negative is padding: it reads no state and writes none.
template <typename OT>
__global__ void __launch_bounds__(THREADS)
mingru_direct_kernel(Rows in, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ slots, float* __restrict__ state,
                     long long state_stride, OT* __restrict__ out, int W) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const int c = blockIdx.x * THREADS + threadIdx.x;
  if (c >= W) return;
  const int r = blockIdx.y;
  const int slot = slots[r];
  const float bz = in.bz ? in.bz[c] : 0.f, bu = in.bu ? in.bu[c] : 0.f;
  float S = slot >= 0 ? state[slot * state_stride + c] : 0.f;
  S = walk<OT>(in, cu_q[r], cu_q[r + 1], c, bz, bu, S, out, W);
  if (slot >= 0) state[slot * state_stride + c] = S;
}

// grid (ceil(W / THREADS), requests, stretches): (P, B) of every stretch into `parts [R, stretches, 2, W]`;
// the first stretch's block also copies the request's incoming state to `start [R, W]`, so that
// the second kernel, whose last stretch overwrites the state, reads nothing that it writes.
__global__ void __launch_bounds__(THREADS)
mingru_parts_kernel(Rows in, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ slots, const float* __restrict__ state,
                    long long state_stride, float* __restrict__ parts, float* __restrict__ start, int W, int stretches) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const int c = blockIdx.x * THREADS + threadIdx.x;
  if (c >= W) return;
  const int r = blockIdx.y, s = blockIdx.z;
  const int end = cu_q[r + 1];
  const int t0 = cu_q[r] + s * SEG;
  if (s == 0) {
    const int slot = slots[r];
    start[(size_t)r * W + c] = slot >= 0 ? state[slot * state_stride + c] : 0.f;
  }
  if (t0 >= end) return;
  const int t1 = min(end, t0 + SEG);
  const float bz = in.bz ? in.bz[c] : 0.f, bu = in.bu ? in.bu[c] : 0.f;
  float P = 1.f, B = 0.f;
  int t = t0;
  for (; t + AHEAD <= t1; t += AHEAD) {
    float a[AHEAD], u[AHEAD];
#pragma unroll
    for (int k = 0; k < AHEAD; ++k) {
      const float* row = in.proj + (long long)(t + k) * in.stride;
      a[k] = row[in.z_col + c];
      u[k] = row[in.u_col + c];
    }
#pragma unroll
    for (int k = 0; k < AHEAD; ++k) {
      const float z = sigmoidf_(a[k] + bz), v = u[k] + bu;
      const float n = v >= 0.f ? v + 0.5f : sigmoidf_(v);
      P *= 1.0f - z;
      B = fmaf(1.0f - z, B, z * n);
    }
  }
  for (; t < t1; ++t) {
    float p, b;
    gates(in, t, c, bz, bu, p, b);
    P *= p;
    B = fmaf(p, B, b);
  }
  float* o = parts + ((size_t)r * stretches + s) * 2 * W;
  o[c] = P;
  o[W + c] = B;
}

template <typename OT>
__global__ void __launch_bounds__(THREADS)
mingru_finish_kernel(Rows in, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ slots, float* __restrict__ state,
                     long long state_stride, const float* __restrict__ parts, const float* __restrict__ start,
                     OT* __restrict__ out, int W, int stretches) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const int c = blockIdx.x * THREADS + threadIdx.x;
  if (c >= W) return;
  const int r = blockIdx.y, s = blockIdx.z;
  const int end = cu_q[r + 1];
  const int t0 = cu_q[r] + s * SEG;
  if (t0 >= end) return;
  const int t1 = min(end, t0 + SEG);
  float S = start[(size_t)r * W + c];
  const float* pr = parts + (size_t)r * stretches * 2 * W;
  for (int k = 0; k < s; ++k) S = fmaf(pr[(size_t)k * 2 * W + c], S, pr[(size_t)k * 2 * W + W + c]);
  const float bz = in.bz ? in.bz[c] : 0.f, bu = in.bu ? in.bu[c] : 0.f;
  S = walk<OT>(in, t0, t1, c, bz, bu, S, out, W);
  const int slot = slots[r];
  if (t1 == end && slot >= 0) state[slot * state_stride + c] = S;
}

}  // namespace

// How many floats of scratch gb_mingru wants for a step whose longest request brings max_q tokens.
GB_EXPORT long long gb_mingru_scratch_floats(int R, int W, int max_q) {
  if (max_q <= SEG) return 0;
  const long long stretches = (max_q + SEG - 1) / SEG;
  return (long long)R * W * (2 * stretches + 1);
}

// proj [T, stride] 32-bit with the gate's, the candidate's and the output gate's logits at z_col, u_col,
// g_col (W wide each); bz, bu [W] 32-bit or null; state [slots, state_stride] 32-bit, its first W
// entries a request's S; out [T, W] in its dtype. max_q: the longest request's tokens in this step.
GB_EXPORT int gb_mingru(const float* proj, long long stride, int z_col, int u_col, int g_col, const float* bz, const float* bu,
                        const int32_t* cu_q, const int32_t* slots, float* state, long long state_stride, void* out,
                        int out_dtype, int R, int W, int max_q, float* scratch, cudaStream_t stream) {
  if (R <= 0 || W <= 0) return GB_OK;
  if (R > 65535) return gb::fail(GB_UNSUPPORTED, "mingru: %d requests (at most 65535 a step)", R);
  const Rows in = {proj, stride, z_col, u_col, g_col, bz, bu};
  const int blocks = (W + THREADS - 1) / THREADS;
  return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
    if (max_q <= SEG)
      return gb::check_pdl_launch(gb::launch_pdl(mingru_direct_kernel<OT>, dim3(blocks, R), dim3(THREADS), 0, stream,
                                                 dim3(1, 1, 1), in, cu_q, slots, state, state_stride, (OT*)out, W),
                                  "mingru");
    const int stretches = (max_q + SEG - 1) / SEG;
    if (stretches > 65535) return gb::fail(GB_UNSUPPORTED, "mingru: %d tokens of one request in a step", max_q);
    if (scratch == nullptr) return gb::fail(GB_BAD_ARGUMENT, "mingru: a step this long needs scratch");
    float* parts = scratch;
    float* start = scratch + (size_t)R * stretches * 2 * W;
    const dim3 grid(blocks, R, stretches);
    int rc = gb::check_pdl_launch(gb::launch_pdl(mingru_parts_kernel, grid, dim3(THREADS), 0, stream, dim3(1, 1, 1), in, cu_q,
                                                 slots, (const float*)state, state_stride, parts, start, W, stretches),
                                  "mingru_parts");
    if (rc != GB_OK) return rc;
    return gb::check_pdl_launch(gb::launch_pdl(mingru_finish_kernel<OT>, grid, dim3(THREADS), 0, stream, dim3(1, 1, 1), in, cu_q,
                                               slots, state, state_stride, (const float*)parts, (const float*)start, (OT*)out,
                                               W, stretches),
                                "mingru_finish");
  });
}
