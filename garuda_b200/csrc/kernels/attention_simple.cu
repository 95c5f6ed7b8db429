// Causal grouped-query attention over the paged cache, one warp per (token,
// query head), 32-bit arithmetic throughout: the attention of the 32-bit path
// and the check beside the tensor-core kernel.
//
// garuda/src/llama/mod.rs:793-818: query head h reads kv head h / g; score
// s_j = dot(q, K_j) * scale with the scale multiplied after the dot; keys j in
// [start, pos], start = max(0, pos + 1 - window) (garuda/src/cache/mod.rs:333-338);
// softmax with the maximum subtracted (garuda/src/simd/mod.rs:132-158); then the
// sum of p_j V_j in key order. Keys are walked 32 at a time from `start`, with
// a running maximum and sum, so the result for a token does not depend on what
// else is in the batch or on how its prompt was cut.
//
// Options that other designs use, each off at its neutral value: `softcap` c > 0 replaces a score
// by c tanh(s / c) (after the scale); `keep_first` n > 0 lets a windowed query also read the first
// n positions of its request (at their true positions); `sink` adds one to the softmax's
// denominator, an entry of score zero that carries no value: p_j = exp(s_j) / (1 + sum exp(s_k));
// `sink_v` (one learned number per query head) adds exp(sink_v[h]) there instead, unscaled; `r1`, `r2`
// (per query head) take r1 ln(1 + r2 (i - j)) off the score of key j for the query at i; `chunk` n > 0
// lets a query read only the keys of its own stretch of n positions, floor(j / n) = floor(i / n),
// counted from the request's first position.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;

// MAX_HD: the widest head this instance takes. A value row is `v_hd` wide in its pool, of which the
// first `vd` channels are summed (vd = v_hd = hd for ordinary attention; a mixer whose keys and
// values are parts of one cached vector passes the same pool twice and a narrower vd).
template <typename T, int MAX_HD>
__global__ void __launch_bounds__(WARPS * 32)
attention_simple_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                        const int32_t* __restrict__ block_table, int table_width,
                        const int32_t* __restrict__ cu_q, const int32_t* __restrict__ kv_lens,
                        const int32_t* __restrict__ token_req, T* __restrict__ out, int Hq, int Hkv, int hd,
                        int v_hd, int vd, float scale, int window, int page_size, float softcap, int keep_first,
                        int sink, const float* __restrict__ sink_v, const float* __restrict__ r1,
                        const float* __restrict__ r2, int chunk) {
  __shared__ float q_s[WARPS][MAX_HD];
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * WARPS + warp;
  if (h >= Hq) return;
  const int r = token_req[t];
  const int q_len = cu_q[r + 1] - cu_q[r];
  const int pos = kv_lens[r] - q_len + (t - cu_q[r]);
  const int start = chunk > 0 ? (pos / chunk) * chunk : window > 0 ? max(0, pos + 1 - window) : 0;
  const float far1 = r1 ? r1[h] : 0.f, far2 = r2 ? r2[h] : 0.f;
  const int kvh = h / (Hq / Hkv);
  const int32_t* table = block_table + (size_t)r * table_width;

  const T* qr = q + ((size_t)t * Hq + h) * hd;
  for (int c = lane; c < hd; c += 32) q_s[warp][c] = gb::to_float<T>(qr[c]);
  __syncwarp();

  const int nacc = (vd + 31) / 32;
  float acc[MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  // two stretches of keys: the kept first positions below the window, then the window
  const int kept = start > 0 ? min(keep_first, start) : 0;
  const int n_blocks_kept = (kept + 31) / 32;
  const int n_blocks = n_blocks_kept + (pos - start + 32) / 32;
  for (int blk = 0; blk < n_blocks; ++blk) {
    const bool in_kept = blk < n_blocks_kept;
    const int base = in_kept ? blk * 32 : start + (blk - n_blocks_kept) * 32;
    const int last = in_kept ? kept - 1 : pos;
    const int j = base + lane;
    const bool valid = j <= last;
    long long row = -1;  // row of this lane's key in the pool, in units of hd elements
    if (valid) {
      const int page = table[j / page_size];
      if (page >= 0) row = ((long long)page * Hkv + kvh) * page_size + (j % page_size);
    }
    float s = -INFINITY;
    if (row >= 0) {
      const T* kr = k_pool + row * hd;
      float dot = 0.f;
      for (int c = 0; c < hd; ++c) dot = fmaf(q_s[warp][c], gb::to_float<T>(kr[c]), dot);
      s = dot * scale;
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      if (r1) s -= far1 * log1pf(far2 * (float)(pos - j));
    }
    const float m_new = fmaxf(m, gb::warp_max(s));
    if (m_new == -INFINITY) continue;          // a block without a single stored key
    const float p = row >= 0 ? expf(s - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + gb::warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; ++i) acc[i] *= corr;
    const int n_here = min(32, last - base + 1);
    for (int jj = 0; jj < n_here; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long rj = __shfl_sync(0xffffffffu, row, jj);
      if (rj < 0) continue;
      const T* vr = v_pool + rj * v_hd;
#pragma unroll
      for (int i = 0; i < MAX_HD / 32; ++i) {
        const int c = lane + 32 * i;
        if (i < nacc && c < vd) acc[i] = fmaf(pj, gb::to_float<T>(vr[c]), acc[i]);
      }
    }
  }
  if (sink_v && m != -INFINITY) l += expf(sink_v[h] - m);
  else if (sink && m != -INFINITY) l += expf(-m);
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  T* o = out + ((size_t)t * Hq + h) * vd;
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) {
    const int c = lane + 32 * i;
    if (i < nacc && c < vd) o[c] = gb::from_float<T>(acc[i] * inv);
  }
}

}  // namespace

// v_hd: width of a value row in its pool; vd: how many of its first channels are the value
// (out is [T, Hq, vd]). Ordinary attention passes hd for both.
GB_EXPORT int gb_attention_simple(const void* q, const void* k_pool, const void* v_pool, int dtype,
                                  const int32_t* block_table, int table_width, const int32_t* cu_q,
                                  const int32_t* kv_lens, const int32_t* token_req, void* out, int T,
                                  int Hq, int Hkv, int hd, int v_hd, int vd, float scale, int window,
                                  int page_size, float softcap, int keep_first, int sink, const float* sink_v,
                                  const float* r1, const float* r2, int chunk, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  constexpr int WIDEST = 1024;
  if (hd > WIDEST || hd < 1)
    return gb::fail(GB_UNSUPPORTED, "attention: head_dim %d is outside 1..%d", hd, WIDEST);
  if (vd < 1 || vd > v_hd || vd > WIDEST)
    return gb::fail(GB_BAD_ARGUMENT, "attention: %d value channels of rows %d wide", vd, v_hd);
  if (Hkv < 1 || Hq % Hkv) return gb::fail(GB_BAD_ARGUMENT, "attention: %d query heads for %d kv heads", Hq, Hkv);
  if ((r1 == nullptr) != (r2 == nullptr)) return gb::fail(GB_BAD_ARGUMENT, "attention: the distance term takes both of its numbers");
  if (chunk < 0 || (chunk > 0 && (window > 0 || keep_first > 0)))
    return gb::fail(GB_BAD_ARGUMENT, "attention: a stretch of %d positions goes with no window", chunk);
  dim3 grid(T, (Hq + WARPS - 1) / WARPS);
  return GB_DISPATCH_DTYPE(dtype, TT, [&]() -> int {
    if (hd <= 256 && vd <= 256)
      attention_simple_kernel<TT, 256><<<grid, WARPS * 32, 0, stream>>>(
          (const TT*)q, (const TT*)k_pool, (const TT*)v_pool, block_table, table_width, cu_q, kv_lens,
          token_req, (TT*)out, Hq, Hkv, hd, v_hd, vd, scale, window, page_size, softcap, keep_first, sink, sink_v, r1, r2, chunk);
    else
      attention_simple_kernel<TT, WIDEST><<<grid, WARPS * 32, 0, stream>>>(
          (const TT*)q, (const TT*)k_pool, (const TT*)v_pool, block_table, table_width, cu_q, kv_lens,
          token_req, (TT*)out, Hq, Hkv, hd, v_hd, vd, scale, window, page_size, softcap, keep_first, sink, sink_v, r1, r2, chunk);
    return gb::check_launch("attention_simple");
  });
}
