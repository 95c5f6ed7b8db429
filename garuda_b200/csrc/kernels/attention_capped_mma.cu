// bfloat16 grouped-query attention over the paged cache on the tensor cores (mma.sync m16n8k16,
// 32-bit accumulation), flash-style, for the variants the plain kernels of attention_mma.cu do not
// take: keys and values of widths of their own, scores capped by c tanh(s / c), a window that also
// keeps a request's first positions, and a sink (one more entry of score zero, without a value, in
// the softmax's denominator), or a learned sink per query head (exp(sink_h) there instead of one), a
// term on the scores that grows with the logarithm of the distance, and a mask of fixed stretches
// of positions in place of the window. No position encoding: positions enter through the mask and
// the distance term only.
//
//   s_ij = (q_i . k_j) * scale;   cap c > 0:  s_ij <- c tanh(s_ij / c);   s_ij -= r1_h ln(1 + r2_h (i - j))
//   i reads j  iff  j <= i and (window == 0 or i - j < window or j < keep_first)
//              or, chunk n > 0:  j <= i and floor(j / n) = floor(i / n)
//   p_ij = exp(s_ij - m_i) / (sink exp(-m_i) + sum_j' exp(s_ij' - m_i)),  sink = 1 or exp(sink_h)
//
// Scores, the cap, the running maximum and sum are 32-bit; probabilities are rounded to bfloat16
// only as an operand of the second product. The rows of a query tile are (token, head-of-group)
// pairs of one kv head of one request, so a K/V tile is read once for the whole group. Keys are
// walked in tiles of 64: first the tiles that hold kept first positions below the window, then the
// window's. Two shapes of one kernel:
//  * TILE (prompt portions): 64 rows per CTA, 16 per warp, every warp walks all key tiles.
//  * DECODE (a request with at most 16 rows): the four warps take a quarter of every tile's keys
//    each for the same rows and merge in shared memory; `splits` CTAs share a request's tiles and
//    leave partial results in the caller's scratch, which a second kernel merges in split order.
// A request belongs to DECODE if q_len * g <= 16, else to TILE; each launch skips the other's.
//
// Compiled per (key width, value width): GB_KEY_DIM, GB_VALUE_DIM (multiples of 16, at most 128).
#include "attention_mma_core.cuh"
#include "common.cuh"

#ifndef GB_KEY_DIM
#define GB_KEY_DIM 64
#endif
#ifndef GB_VALUE_DIM
#define GB_VALUE_DIM 64
#endif

namespace {

using namespace attn_mma;

constexpr int HD = GB_KEY_DIM, VD = GB_VALUE_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 128 && VD % 16 == 0 && VD >= 16 && VD <= 128, "widths are multiples of 16 up to 128");
constexpr int PAD = 8;
constexpr int LDK = HD + PAD, LDV = VD + PAD;
constexpr int THREADS = 128;
constexpr int ROWS_TILE = 64, ROWS_DECODE = 16;
constexpr int MAX_SPLITS = 32;
constexpr int PR = VD + 2;                 // floats of a row's partial result: sums, maximum, denominator
constexpr float LOG2E = 1.4426950408889634f;
constexpr size_t SMEM = (size_t)(ROWS_TILE * LDK + 2 * KT * (LDK + LDV)) * sizeof(__nv_bfloat16);

struct Params {
  const __nv_bfloat16* q;        // [T, Hq, HD]
  const __nv_bfloat16* k_pool;   // [pages, Hkv, page_size, HD]
  const __nv_bfloat16* v_pool;   // [pages, Hkv, page_size, VD]
  __nv_bfloat16* out;            // [T, Hq * VD]
  const int32_t* block_table;
  const int32_t* cu_q;
  const int32_t* kv_lens;
  float* partials;               // [R, Hkv, splits, ROWS_DECODE, PR] (DECODE with splits > 1)
  int table_width, Hq, Hkv, g, window, keep_first, page_size, sink, splits;
  float scale, softcap;
  const float* sink_v;           // [Hq] or null: a learned sink per query head
  const float* r1;               // [Hq] or null: the distance term's two numbers per query head
  const float* r2;
  int chunk;                     // > 0: a query reads its own stretch of this many positions (no window then)
};

// First position that the query at `pos` reads (kept first positions aside).
__device__ __forceinline__ int first_seen(const Params& p, int pos) {
  if (p.chunk > 0) return pos / p.chunk * p.chunk;
  return p.window > 0 ? max(0, pos + 1 - p.window) : 0;
}

// What the sink adds to a row's denominator, in units of exp(-m).
__device__ __forceinline__ float sink_term(const Params& p, int head, float m) {
  if (m == -INFINITY) return 0.f;
  if (p.sink_v != nullptr) return fast_exp2((p.sink_v[head] - m) * 1.4426950408889634f);
  return p.sink ? fast_exp2(-m * 1.4426950408889634f) : 0.f;
}

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// tanh by way of the exponential: 1 - 2 / (2^(2 x log2 e) + 1); absolute error about 2^-22
__device__ __forceinline__ float tanh_exp2(float x) {
  x = fminf(fmaxf(x, -15.f), 15.f);          // tanh(15) is 1 to 32-bit accuracy
  const float t = fast_exp2(x * (2.0f * LOG2E));
  return 1.0f - __fdividef(2.0f, t + 1.0f);
}

// tanh(x): within [-1, 1] (a score below its cap, the usual case) an odd polynomial of degree 13 on
// the multiply-add units, fitted to tanh on that interval (largest error 9e-8 as evaluated in
// 32-bit, an ulp of the values near one), which leaves the special-function unit to the softmax's
// exponential; beyond it the exponential form, which a warp takes for a tile only if one of its
// scores is there (one test per tile, not per score).
__device__ __forceinline__ float tanh_poly(float x, float x2) {
  float q = 0.0009637729963287711f;
  q = fmaf(q, x2, -0.005951283033937216f);
  q = fmaf(q, x2, 0.019973287358880043f);
  q = fmaf(q, x2, -0.05326583608984947f);
  q = fmaf(q, x2, 0.13319583237171173f);
  q = fmaf(q, x2, -0.33332130312919617f);
  q = fmaf(q, x2, 0.9999997019767761f);
  return q * x;
}

// The CTA copies keys [tile_start, tile_start + 64) of one kv head, keys and values, 16 bytes per
// copy; a key's page is looked up by the thread that copies its first chunk and handed round in
// shared memory. Keys outside [lo, hi] that are not among the first `keep`, or without a page, become zeros (an unwritten or reused page
// may hold anything, and a probability of zero times a NaN is a NaN).
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* ks, __nv_bfloat16* vs, int64_t* where, const Params& p,
                                             const int32_t* table, int kvh, int tile_start, int lo, int hi, int keep) {
  __syncthreads();        // the copies of the tile in front have read `where`
  if (threadIdx.x < KT) {
    const int j = tile_start + threadIdx.x;
    int64_t w = -1;
    if (j <= hi && (j >= lo || j < keep)) {        // in the window, or a kept first position
      const int page = table[j / p.page_size];
      if (page >= 0) w = ((int64_t)page * p.Hkv + kvh) * p.page_size + (j % p.page_size);
    }
    where[threadIdx.x] = w;
  }
  __syncthreads();
  constexpr int CK = HD / 8, CV = VD / 8;
  for (int c = threadIdx.x; c < KT * CK; c += THREADS) {
    const int row = c / CK, ch = c % CK;
    const int64_t w = where[row];
    cp_async_16(ks + row * LDK + ch * 8, p.k_pool + (w >= 0 ? (size_t)w * HD + ch * 8 : 0), w >= 0);
  }
  for (int c = threadIdx.x; c < KT * CV; c += THREADS) {
    const int row = c / CV, ch = c % CV;
    const int64_t w = where[row];
    cp_async_16(vs + row * LDV + ch * 8, p.v_pool + (w >= 0 ? (size_t)w * VD + ch * 8 : 0), w >= 0);
  }
}

struct State {
  float o[VD / 8][4];
  float m[2], l[2];              // the maximum in the units of the capped, scaled score
};

// KEYS keys (from column key_off of the tile) for one warp's 16 rows. MASKED false: every key of the
// tile is seen by every row (no comparison per score).
// FAR: the distance term, far1 ln(1 + far2 (i - j)) with the row's head's numbers, is taken off.
template <int KEYS, bool MASKED, bool FAR>
__device__ __forceinline__ void process(State& st, const uint32_t (&qf)[HD / 16][4], const __nv_bfloat16* ks,
                                        const __nv_bfloat16* vs, int key_off, int key0, const int (&row_pos)[2],
                                        const int (&row_start)[2], const float (&far1)[2], const float (&far2)[2],
                                        const Params& p) {
  const int lane = threadIdx.x & 31;
  float s[KEYS / 8][4];
#pragma unroll
  for (int n = 0; n < KEYS / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
    for (int n2 = 0; n2 < KEYS / 16; ++n2) {
      uint32_t b[4];
      const int key = key_off + n2 * 16 + (lane % 8) + (lane / 16) * 8;
      ldmatrix_x4(b, ks + key * LDK + (kk * 2 + ((lane / 8) % 2)) * 8);
      mma_16816(s[2 * n2], qf[kk], b[0], b[1]);
      mma_16816(s[2 * n2 + 1], qf[kk], b[2], b[3]);
    }
  }
  float m_new[2] = {st.m[0], st.m[1]};
  const bool capped = p.softcap > 0.f;
  const float pre = capped ? p.scale / p.softcap : p.scale, post = capped ? p.softcap : 1.0f;
  if (capped) {
    float largest = 0.f;
#pragma unroll
    for (int n = 0; n < KEYS / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) largest = fmaxf(largest, fabsf(s[n][e]));
    if (__any_sync(0xffffffffu, largest * pre > 1.0f)) {       // rare: a score beyond its cap
#pragma unroll
      for (int n = 0; n < KEYS / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float v = s[n][e] * pre, v2 = v * v;
          s[n][e] = post * (v2 > 1.0f ? tanh_exp2(v) : tanh_poly(v, v2));
        }
    } else {
#pragma unroll
      for (int n = 0; n < KEYS / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float v = s[n][e] * pre;
          s[n][e] = post * tanh_poly(v, v * v);
        }
    }
  } else {
#pragma unroll
    for (int n = 0; n < KEYS / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] *= pre;
  }
#pragma unroll
  for (int n = 0; n < KEYS / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = e >> 1;
      float v = s[n][e];
      const int j = key0 + key_off + n * 8 + (lane % 4) * 2 + (e & 1);
      if (FAR) {
        // ln(1 + x) = log2(1 + x) ln 2; a key behind the row (masked below) is given distance zero
        const float dist = (float)max(row_pos[i] - j, 0);
        v -= far1[i] * __log2f(fmaf(far2[i], dist, 1.0f));
        s[n][e] = v;
      }
      if (MASKED) {
        const bool seen = j <= row_pos[i] && (j >= row_start[i] || j < p.keep_first);
        v = seen ? v : -INFINITY;
        s[n][e] = v;
      }
      m_new[i] = fmaxf(m_new[i], v);
    }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
    m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
  }
  float corr[2], neg_m[2], l_add[2] = {0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float m_use = m_new[i] == -INFINITY ? 0.f : m_new[i];
    corr[i] = st.m[i] == -INFINITY ? 0.f : fast_exp2((st.m[i] - m_use) * LOG2E);
    neg_m[i] = -m_use * LOG2E;
    st.m[i] = m_new[i];
  }
  uint32_t pf[KEYS / 16][4];
#pragma unroll
  for (int n = 0; n < KEYS / 8; ++n) {
    float pr[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      pr[e] = fast_exp2(fmaf(s[n][e], LOG2E, neg_m[e >> 1]));
      l_add[e >> 1] += pr[e];
    }
    pf[n / 2][(n % 2) * 2 + 0] = pack_bf16(pr[0], pr[1]);
    pf[n / 2][(n % 2) * 2 + 1] = pack_bf16(pr[2], pr[3]);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) st.l[i] = st.l[i] * corr[i] + l_add[i];
#pragma unroll
  for (int n = 0; n < VD / 8; ++n) {
    st.o[n][0] *= corr[0]; st.o[n][1] *= corr[0];
    st.o[n][2] *= corr[1]; st.o[n][3] *= corr[1];
  }
#pragma unroll
  for (int kk = 0; kk < KEYS / 16; ++kk) {
#pragma unroll
    for (int n2 = 0; n2 < VD / 16; ++n2) {
      uint32_t b[4];
      const int key = key_off + kk * 16 + (lane % 8) + ((lane / 8) % 2) * 8;
      ldmatrix_x4_trans(b, vs + key * LDV + (n2 * 2 + (lane / 16)) * 8);
      mma_16816(st.o[2 * n2], pf[kk], b[0], b[1]);
      mma_16816(st.o[2 * n2 + 1], pf[kk], b[2], b[3]);
    }
  }
}

// grid (x, Hkv, R): TILE: x a tile of 64 rows of the request; DECODE: x one of p.splits shares of the keys.
template <bool DECODE, bool FAR>
__global__ void __launch_bounds__(THREADS, (HD <= 64 && VD <= 64) ? 4 : 2)
capped_attention_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [ROWS_TILE][LDK]
  __nv_bfloat16* kv = qs + ROWS_TILE * LDK;                          // 2 stages x ([KT][LDK], [KT][LDV])
  __shared__ int64_t where[KT];
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const int r = blockIdx.z, kvh = blockIdx.y;
  const int q_begin = p.cu_q[r], q_len = p.cu_q[r + 1] - q_begin;
  const bool small = q_len * p.g <= ROWS_DECODE;
  if (small != DECODE || q_len <= 0) return;
  const int tokens_per_tile = DECODE ? q_len : ROWS_TILE / p.g;
  const int tok0 = DECODE ? 0 : blockIdx.x * tokens_per_tile;
  if (tok0 >= q_len) return;
  const int kv_len = p.kv_lens[r];
  const int32_t* table = p.block_table + (size_t)r * p.table_width;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntok = min(tokens_per_tile, q_len - tok0);
  const int nrows = ntok * p.g;
  const int pos0 = kv_len - q_len + tok0;
  const int lo = first_seen(p, pos0);
  const int hi = pos0 + ntok - 1;
  const int last_start = first_seen(p, hi);          // the first position that the tile's last row reads
  const int tile_begin = lo / KT, tile_end = hi / KT + 1;
  // tiles below the window that hold kept first positions
  const int kept_tiles = (p.window > 0 && p.keep_first > 0) ? min((p.keep_first + KT - 1) / KT, tile_begin) : 0;
  const int walk = kept_tiles + tile_end - tile_begin;
  int w_begin = 0, w_end = walk;
  if (DECODE && p.splits > 1) {
    const int per = (walk + p.splits - 1) / p.splits;
    w_begin = min(walk, (int)blockIdx.x * per);
    w_end = min(walk, w_begin + per);
  }
  auto tile_of = [&](int w) { return w < kept_tiles ? w : tile_begin + (w - kept_tiles); };
  auto load = [&](int w, int stage) {
    __nv_bfloat16* ks = kv + stage * KT * (LDK + LDV);
    const bool kept = w < kept_tiles;
    load_kv_tile(ks, ks + KT * LDK, where, p, table, kvh, tile_of(w) * KT, kept ? 0 : lo, kept ? p.keep_first - 1 : hi,
                 p.keep_first);
  };

  // queries: row = token_local * g + head_of_group
  for (int c = threadIdx.x; c < ROWS_TILE * (HD / 8); c += THREADS) {
    const int row = c / (HD / 8), ch = c % (HD / 8);
    const bool valid = row < nrows;
    const int tok = valid ? row / p.g : 0, gh = valid ? row % p.g : 0;
    cp_async_16(qs + row * LDK + ch * 8, p.q + ((size_t)(q_begin + tok0 + tok) * p.Hq + kvh * p.g + gh) * HD + ch * 8, valid);
  }
  if (w_begin < w_end) load(w_begin, 0);
  cp_async_commit();

  const int my_rows = DECODE ? 0 : warp * 16;          // first row of the warp's 16
  int row_pos[2], row_start[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = my_rows + lane / 4 + 8 * i;
    row_pos[i] = row < nrows ? pos0 + row / p.g : -1;
    row_start[i] = row < nrows ? first_seen(p, row_pos[i]) : 0;
  }
  float far1[2] = {0.f, 0.f}, far2[2] = {0.f, 0.f};
  if (FAR) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = my_rows + lane / 4 + 8 * i;
      const int head = kvh * p.g + (row < nrows ? row % p.g : 0);
      far1[i] = p.r1[head] * 0.6931471805599453f;
      far2[i] = p.r2[head];
    }
  }
  State st;
#pragma unroll
  for (int n = 0; n < VD / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) st.o[n][e] = 0.f;
  st.m[0] = st.m[1] = -INFINITY;
  st.l[0] = st.l[1] = 0.f;
  uint32_t qf[HD / 16][4];
  const bool works = DECODE || my_rows < nrows;       // a warp whose rows are all padding only copies
  for (int w = w_begin; w < w_end; ++w) {
    const int stage = (w - w_begin) & 1;
    const __nv_bfloat16* ks = kv + stage * KT * (LDK + LDV);
    const __nv_bfloat16* vs = ks + KT * LDK;
    if (w + 1 < w_end) load(w + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (w == w_begin) {
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk)
        ldmatrix_x4(qf[kk], qs + (my_rows + (lane % 16)) * LDK + kk * 16 + (lane / 16) * 8);
    }
    if (works) {
      // no mask where the tile lies wholly before the first row's position and inside the last row's window
      const int t0 = tile_of(w) * KT;
      const bool full = w >= kept_tiles && t0 + KT - 1 <= pos0 && t0 >= last_start;
      if (DECODE) {
        if (full) process<16, false, FAR>(st, qf, ks, vs, warp * 16, t0, row_pos, row_start, far1, far2, p);
        else process<16, true, FAR>(st, qf, ks, vs, warp * 16, t0, row_pos, row_start, far1, far2, p);
      } else {
        if (full) process<KT, false, FAR>(st, qf, ks, vs, 0, t0, row_pos, row_start, far1, far2, p);
        else process<KT, true, FAR>(st, qf, ks, vs, 0, t0, row_pos, row_start, far1, far2, p);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 1);
    st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 2);
  }
  if (!DECODE) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = my_rows + lane / 4 + 8 * i;
      if (row >= nrows) continue;
      const float l = st.l[i] + sink_term(p, kvh * p.g + row % p.g, st.m[i]);
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      __nv_bfloat16* dst = p.out + ((size_t)(q_begin + tok0 + row / p.g) * p.Hq + kvh * p.g + row % p.g) * VD;
#pragma unroll
      for (int n = 0; n < VD / 8; ++n)
        *reinterpret_cast<uint32_t*>(dst + n * 8 + (lane % 4) * 2) = pack_bf16(st.o[n][2 * i] * inv, st.o[n][2 * i + 1] * inv);
    }
    return;
  }
  // DECODE: the four warps' states over their quarters of the keys, merged in warp order
  __syncthreads();
  float* part = reinterpret_cast<float*>(smem_raw);       // [4][ROWS_DECODE][PR], over the tiles (no longer read)
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = lane / 4 + 8 * i;
    float* pr = part + ((size_t)warp * ROWS_DECODE + row) * PR;
#pragma unroll
    for (int n = 0; n < VD / 8; ++n) {
      pr[n * 8 + (lane % 4) * 2] = st.o[n][2 * i];
      pr[n * 8 + (lane % 4) * 2 + 1] = st.o[n][2 * i + 1];
    }
    if (lane % 4 == 0) {
      pr[VD] = st.m[i];
      pr[VD + 1] = st.l[i];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < ROWS_DECODE * VD; idx += THREADS) {
    const int row = idx / VD, c = idx % VD;
    if (row >= nrows) continue;
    float m = -INFINITY;
    for (int w = 0; w < 4; ++w) m = fmaxf(m, part[((size_t)w * ROWS_DECODE + row) * PR + VD]);
    float o = 0.f, l = 0.f;
    for (int w = 0; w < 4; ++w) {
      const float* pr = part + ((size_t)w * ROWS_DECODE + row) * PR;
      const float f = pr[VD] == -INFINITY ? 0.f : fast_exp2((pr[VD] - m) * LOG2E);
      o = fmaf(pr[c], f, o);
      l = fmaf(pr[VD + 1], f, l);
    }
    if (p.splits > 1) {
      float* dst = p.partials + ((((size_t)r * p.Hkv + kvh) * p.splits + blockIdx.x) * ROWS_DECODE + row) * PR;
      dst[c] = o;
      if (c == 0) {
        dst[VD] = m;
        dst[VD + 1] = l;
      }
    } else {
      l += sink_term(p, kvh * p.g + row % p.g, m);
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      p.out[((size_t)(q_begin + row / p.g) * p.Hq + kvh * p.g + row % p.g) * VD + c] = __float2bfloat16_rn(o * inv);
    }
  }
}

// grid (Hkv, R): the shares of a decode request's keys, merged in split order; the sink joins here.
__global__ void __launch_bounds__(THREADS)
capped_attention_merge_kernel(const Params p) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const int kvh = blockIdx.x, r = blockIdx.y;
  const int q_begin = p.cu_q[r], q_len = p.cu_q[r + 1] - q_begin;
  if (q_len * p.g > ROWS_DECODE || q_len <= 0) return;
  const int nrows = q_len * p.g;
  const float* base = p.partials + ((size_t)r * p.Hkv + kvh) * p.splits * ROWS_DECODE * PR;
  for (int idx = threadIdx.x; idx < nrows * VD; idx += THREADS) {
    const int row = idx / VD, c = idx % VD;
    float m = -INFINITY;
    for (int s = 0; s < p.splits; ++s) m = fmaxf(m, base[((size_t)s * ROWS_DECODE + row) * PR + VD]);
    float o = 0.f, l = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const float* pr = base + ((size_t)s * ROWS_DECODE + row) * PR;
      const float f = pr[VD] == -INFINITY ? 0.f : fast_exp2((pr[VD] - m) * LOG2E);
      o = fmaf(pr[c], f, o);
      l = fmaf(pr[VD + 1], f, l);
    }
    l += sink_term(p, kvh * p.g + row % p.g, m);
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    p.out[((size_t)(q_begin + row / p.g) * p.Hq + kvh * p.g + row % p.g) * VD + c] = __float2bfloat16_rn(o * inv);
  }
}

}  // namespace

GB_DEFINE_LAST_ERROR()

GB_EXPORT int gb_capped_attention_key_dim() { return HD; }
GB_EXPORT int gb_capped_attention_value_dim() { return VD; }

// Bytes of scratch for `splits` CTAs per decode request (0 for one).
GB_EXPORT long long gb_capped_attention_scratch_bytes(int R, int kv_heads, int splits) {
  return splits > 1 ? (long long)R * kv_heads * splits * ROWS_DECODE * PR * (long long)sizeof(float) : 0;
}

// q [T, Hq, HD], k_pool [pages, Hkv, page_size, HD], v_pool [pages, Hkv, page_size, VD], out [T, Hq * VD],
// bfloat16. A split that holds no key of a request leaves a partial with maximum -inf, which the merge skips.
GB_EXPORT int gb_capped_attention(const void* q, const void* k_pool, const void* v_pool, void* out,
                                  const int32_t* block_table, int table_width, const int32_t* cu_q,
                                  const int32_t* kv_lens, int T, int R, int Hq, int Hkv, float scale, float softcap,
                                  int window, int keep_first, int sink, int page_size, int max_q_len, int min_q_len,
                                  int splits, void* scratch, long long scratch_bytes, const float* sink_v, const float* r1,
                                  const float* r2, int chunk, cudaStream_t stream) {
  if (T <= 0 || R <= 0) return GB_OK;
  if (Hkv < 1 || Hq % Hkv) return gb::fail(GB_BAD_ARGUMENT, "capped_attention: %d query heads for %d kv heads", Hq, Hkv);
  if ((r1 == nullptr) != (r2 == nullptr)) return gb::fail(GB_BAD_ARGUMENT, "capped_attention: the distance term takes both of its numbers");
  if (chunk < 0 || (chunk > 0 && window > 0)) return gb::fail(GB_BAD_ARGUMENT, "capped_attention: a stretch of %d positions goes with no window", chunk);
  const int g = Hq / Hkv;
  if (g > ROWS_TILE) return gb::fail(GB_UNSUPPORTED, "capped_attention: a group of %d query heads per kv head", g);
  splits = splits < 1 ? 1 : (splits > MAX_SPLITS ? MAX_SPLITS : splits);
  if (splits > 1 && (scratch == nullptr || scratch_bytes < gb_capped_attention_scratch_bytes(R, Hkv, splits)))
    return gb::fail(GB_BAD_ARGUMENT, "capped_attention: %d splits need more scratch", splits);
  Params p;
  p.q = (const __nv_bfloat16*)q; p.k_pool = (const __nv_bfloat16*)k_pool; p.v_pool = (const __nv_bfloat16*)v_pool;
  p.out = (__nv_bfloat16*)out; p.block_table = block_table; p.cu_q = cu_q; p.kv_lens = kv_lens;
  p.partials = (float*)scratch;
  p.table_width = table_width; p.Hq = Hq; p.Hkv = Hkv; p.g = g; p.window = window;
  p.keep_first = window > 0 ? keep_first : 0; p.page_size = page_size; p.sink = sink; p.splits = splits;
  p.scale = scale; p.softcap = softcap;
  p.sink_v = sink_v; p.r1 = r1; p.r2 = r2; p.chunk = chunk;
  const bool far = r1 != nullptr;
  auto decode_kernel = far ? capped_attention_kernel<true, true> : capped_attention_kernel<true, false>;
  auto tile_kernel = far ? capped_attention_kernel<false, true> : capped_attention_kernel<false, false>;
  static gb::OncePerDevice configured;
  if (configured.needed()) {
    cudaError_t e = cudaSuccess;
    for (auto k : {capped_attention_kernel<false, false>, capped_attention_kernel<true, false>,
                   capped_attention_kernel<false, true>, capped_attention_kernel<true, true>}) {
      const cudaError_t e1 = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
      if (e1 != cudaSuccess) e = e1;
    }
    if (e != cudaSuccess) return gb::fail(GB_CUDA_ERROR, "capped_attention: %s", cudaGetErrorString(e));
    configured.done();
  }
  if (min_q_len * g <= ROWS_DECODE) {
    int rc = gb::check_pdl_launch(gb::launch_pdl(decode_kernel, dim3(splits, Hkv, R), dim3(THREADS), SMEM,
                                                 stream, dim3(1, 1, 1), p), "capped_attention (decode)");
    if (rc) return rc;
    if (splits > 1) {
      rc = gb::check_pdl_launch(gb::launch_pdl(capped_attention_merge_kernel, dim3(Hkv, R), dim3(THREADS), 0, stream,
                                               dim3(1, 1, 1), p), "capped_attention (merge)");
      if (rc) return rc;
    }
  }
  if (max_q_len * g > ROWS_DECODE) {
    const int tokens_per_tile = ROWS_TILE / g;
    dim3 grid((max_q_len + tokens_per_tile - 1) / tokens_per_tile, Hkv, R);
    return gb::check_pdl_launch(gb::launch_pdl(tile_kernel, grid, dim3(THREADS), SMEM, stream,
                                               dim3(1, 1, 1), p), "capped_attention (tile)");
  }
  return GB_OK;
}
