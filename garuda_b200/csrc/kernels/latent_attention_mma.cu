// Causal attention over cached latent rows on the tensor cores (bfloat16, mma.sync.m16n8k16,
// 32-bit accumulators and softmax), compiled for one (RANK, ROT) at a time.
//
// Every position has one cached row [c (RANK) | r (ROT)] that all H heads read; a query row is
// [W_uk^T q^n (RANK) | q^r (ROT)]. Scores are dots over the whole row, values are the row's first
// RANK channels:
//     s_ij = (q_i . row_j) * scale,  o_i = sum_j softmax_j(s_ij) row_j[0:RANK]
// The query rows of a request are its (token, head) pairs in that order, which is also the order
// of q's and out's rows in memory, so a tile of 64 query rows is 64 consecutive rows: with H
// heads, a key tile brought into shared memory serves 64 / H tokens times H heads at once, which
// is the point of keeping one row per position (the cache is read once per tile, not per head).
//
// A CTA: 64 query rows (four row blocks of 16), tiles of 32 keys through a two-stage cp.async
// ring. A warp owns one row block and VCOLS of the value columns; with RANK > 256 (an accumulator
// too large for one warp's registers) two warps share a row block: each computes the scores of 16
// of a tile's 32 keys and half of the value columns, and they exchange the rows' maxima and the
// probabilities (as packed A fragments, which are laid out alike in both warps) through shared
// memory, meeting at a barrier of their own. Keys may be split over CTAs (grid.z): every CTA then writes unnormalised
// sums with its running maximum and denominator, and a second kernel merges them in split order.
// A masked key's row is zero-filled in shared memory, so that whatever lies in pages not yet
// written (NaN included) never reaches a sum.
#include "attention_mma_core.cuh"
#include "common.cuh"

#if !defined(GB_LATENT_RANK) || !defined(GB_LATENT_ROT)
#error "compile with -DGB_LATENT_RANK=<rank> -DGB_LATENT_ROT=<rot>"
#endif

GB_DEFINE_LAST_ERROR()

namespace {

using attn_mma::fast_exp2;
using attn_mma::ldmatrix_x4;
using attn_mma::ldmatrix_x4_trans;
using attn_mma::mma_16816;
using attn_mma::pack_bf16;

constexpr int RANK = GB_LATENT_RANK, ROT = GB_LATENT_ROT, ROW = RANK + ROT;
constexpr int NSPLIT = RANK > 256 ? 2 : 1;       // warps that share a row block
constexpr int VCOLS = RANK / NSPLIT;             // value columns per warp
constexpr int BM = 64, BN = 32;
constexpr int THREADS = 128 * NSPLIT;
constexpr int PITCH = ROW * 2 + 16;              // bytes; an odd number of 16-byte chunks: ldmatrix without conflicts
constexpr int CHUNKS = ROW / 8;                  // 16-byte chunks of a row
constexpr int LPR = THREADS / BN;                // threads that copy one key row
constexpr size_t SMEM = (size_t)(BM + 2 * BN) * PITCH;
static_assert(ROW % 16 == 0 && RANK % (16 * NSPLIT) == 0 && RANK >= 16 && RANK <= 512, "unsupported latent sizes");
static_assert(SMEM <= 227 * 1024, "the tiles do not fit the shared memory");

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int n = valid ? 16 : 0;                  // 0: the sixteen bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(THREADS, 1)
latent_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pool,
                        __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                        const int32_t* __restrict__ block_table, int table_width, const int32_t* __restrict__ cu_q,
                        const int32_t* __restrict__ kv_lens, int H, float sc, int page_size, int splits,
                        const float* __restrict__ sink_v) {
  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char* q_s = smem;
  unsigned char* k_s = smem + BM * PITCH;
  const int r = blockIdx.y, split = blockIdx.z;
  const int q0 = cu_q[r], q_len = cu_q[r + 1] - q0, kv_len = kv_lens[r];
  const int rows = q_len * H, row0 = blockIdx.x * BM;
  if (row0 >= rows) return;
  const int rows_here = min(BM, rows - row0);
  const int start_pos = kv_len - q_len;
  const int limit = start_pos + (row0 + rows_here - 1) / H + 1;      // this tile's rows read keys [0, limit)
  int k_begin = 0, k_end = limit;
  if (splits > 1) {
    const int chunk = ((limit + splits - 1) / splits + BN - 1) / BN * BN;
    k_begin = min(limit, split * chunk);
    k_end = min(limit, k_begin + chunk);
  }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rb = warp / NSPLIT, cs = warp % NSPLIT;
  const int g = lane >> 2, tig = lane & 3;
  const int32_t* table = block_table + (size_t)r * table_width;
  const size_t grow0 = (size_t)q0 * H + row0;                        // first row of the tile in q and out
  const int n_tiles = (k_end - k_begin + BN - 1) / BN;

  // the query tile, and the first key tile behind it in the same group
  for (int idx = tid; idx < BM * CHUNKS; idx += THREADS) {
    const int rr = idx / CHUNKS, ch = idx % CHUNKS;
    const bool valid = rr < rows_here;
    cp_async16(q_s + rr * PITCH + ch * 16, q + (grow0 + (valid ? rr : 0)) * ROW + ch * 8, valid);
  }
  auto load_keys = [&](int kt, int stage) {
    const int kr = tid / LPR;
    const int j = k_begin + kt * BN + kr;
    int page = -1;
    if (j < k_end) page = table[j / page_size];
    const bool valid = page >= 0;
    const __nv_bfloat16* src = pool + ((size_t)(valid ? page : 0) * page_size + (valid ? j % page_size : 0)) * ROW;
    unsigned char* dst = k_s + ((size_t)stage * BN + kr) * PITCH;
    for (int ch = tid % LPR; ch < CHUNKS; ch += LPR) cp_async16(dst + ch * 16, src + ch * 8, valid);
  };
  if (n_tiles > 0) load_keys(0, 0);
  cp_async_commit();

  float o[VCOLS / 8][4];
#pragma unroll
  for (int n = 0; n < VCOLS / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int i0 = row0 + rb * 16 + g, i1 = i0 + 8;                    // the thread's two rows within the request
  const int qpos0 = i0 < rows ? start_pos + i0 / H : -1;
  const int qpos1 = i1 < rows ? start_pos + i1 / H : -1;
  const bool active = rb * 16 < rows_here;
  // what the two warps of a row block exchange (NSPLIT == 2)
  __shared__ float x_max[4][2][16], x_sum[4][2][16];
  __shared__ uint4 x_p[4][2][32];
  auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + rb) : "memory"); };
  constexpr int SN = NSPLIT == 2 ? 1 : 2;          // blocks of 16 keys whose scores this warp computes

  for (int kt = 0; kt < n_tiles; ++kt) {
    if (kt + 1 < n_tiles) load_keys(kt + 1, (kt + 1) & 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (active) {
      const unsigned char* kst = k_s + (size_t)(kt & 1) * BN * PITCH;
      float s[2 * SN][4];
#pragma unroll
      for (int n = 0; n < 2 * SN; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
#pragma unroll 4
      for (int k0 = 0; k0 < ROW; k0 += 16) {
        uint32_t a[4];
        ldmatrix_x4(a, q_s + (rb * 16 + (lane & 15)) * PITCH + (k0 + (lane >> 4) * 8) * 2);
#pragma unroll
        for (int i = 0; i < SN; ++i) {
          const int np = NSPLIT == 2 ? cs : i;
          uint32_t b[4];
          ldmatrix_x4(b, kst + (np * 16 + (lane & 7) + ((lane >> 4) << 3)) * PITCH + (k0 + ((lane >> 3) & 1) * 8) * 2);
          mma_16816(s[2 * i], a, b[0], b[1]);
          mma_16816(s[2 * i + 1], a, b[2], b[3]);
        }
      }
      const int kbase = k_begin + kt * BN;
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < 2 * SN; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = kbase + (NSPLIT == 2 ? cs * 16 : 0) + n * 8 + 2 * tig + (e & 1);
          const int qp = e < 2 ? qpos0 : qpos1;
          const float t = (key > qp || key >= k_end) ? -INFINITY : s[n][e] * sc;
          s[n][e] = t;
          if (e < 2) mx0 = fmaxf(mx0, t); else mx1 = fmaxf(mx1, t);
        }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      if (NSPLIT == 2) {
        if (tig == 0) {
          x_max[rb][cs][g] = mx0;
          x_max[rb][cs][g + 8] = mx1;
        }
        pair_sync();
        mx0 = fmaxf(mx0, x_max[rb][cs ^ 1][g]);
        mx1 = fmaxf(mx1, x_max[rb][cs ^ 1][g + 8]);
      }
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
      const float c0 = fast_exp2(m0 - ms0), c1 = fast_exp2(m1 - ms1);      // m = -inf: 0
      m0 = mn0;
      m1 = mn1;
      float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
      for (int n = 0; n < 2 * SN; ++n) {
        s[n][0] = fast_exp2(s[n][0] - ms0);
        s[n][1] = fast_exp2(s[n][1] - ms0);
        s[n][2] = fast_exp2(s[n][2] - ms1);
        s[n][3] = fast_exp2(s[n][3] - ms1);
        ps0 += s[n][0] + s[n][1];
        ps1 += s[n][2] + s[n][3];
      }
      l0 = l0 * c0 + ps0;          // each thread keeps the sum over its own keys; the quad adds up at the end
      l1 = l1 * c1 + ps1;
#pragma unroll
      for (int n = 0; n < VCOLS / 8; ++n) {
        o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1;
      }
      if (NSPLIT == 2) {      // this warp's probabilities, as the A fragment of its 16 keys, for its partner
        x_p[rb][cs][lane] = make_uint4(pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]),
                                       pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3]));
        pair_sync();
      }
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) {
        uint32_t a[4];
        if (NSPLIT == 2 && kb != cs) {
          const uint4 other = x_p[rb][cs ^ 1][lane];
          a[0] = other.x; a[1] = other.y; a[2] = other.z; a[3] = other.w;
        } else {
          const int i = NSPLIT == 2 ? 0 : kb;
          a[0] = pack_bf16(s[2 * i][0], s[2 * i][1]);
          a[1] = pack_bf16(s[2 * i][2], s[2 * i][3]);
          a[2] = pack_bf16(s[2 * i + 1][0], s[2 * i + 1][1]);
          a[3] = pack_bf16(s[2 * i + 1][2], s[2 * i + 1][3]);
        }
#pragma unroll
        for (int cp = 0; cp < VCOLS / 16; ++cp) {
          uint32_t b[4];
          const int col = cs * VCOLS + cp * 16;
          ldmatrix_x4_trans(b, kst + (kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + (col + (lane >> 4) * 8) * 2);
          mma_16816(o[2 * cp], a, b[0], b[1]);
          mma_16816(o[2 * cp + 1], a, b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  if (!active) return;
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (NSPLIT == 2) {          // each warp has summed over its own keys
    if (tig == 0) {
      x_sum[rb][cs][g] = l0;
      x_sum[rb][cs][g + 8] = l1;
    }
    pair_sync();
    l0 += x_sum[rb][cs ^ 1][g];
    l1 += x_sum[rb][cs ^ 1][g + 8];
  }
  const size_t gr0 = grow0 + rb * 16 + g, gr1 = gr0 + 8;
  if (splits == 1) {
    // a learned sink per head: exp(sink_h) in the denominator, without a key or a value (m is in powers of two)
    if (sink_v != nullptr) {
      if (i0 < rows && m0 != -INFINITY) l0 += fast_exp2(sink_v[i0 % H] * 1.4426950408889634f - m0);
      if (i1 < rows && m1 != -INFINITY) l1 += fast_exp2(sink_v[i1 % H] * 1.4426950408889634f - m1);
    }
    const float inv0 = l0 > 0.f ? 1.0f / l0 : 0.f, inv1 = l1 > 0.f ? 1.0f / l1 : 0.f;
#pragma unroll
    for (int n = 0; n < VCOLS / 8; ++n) {
      const int col = cs * VCOLS + n * 8 + 2 * tig;
      if (i0 < rows) *reinterpret_cast<uint32_t*>(out + gr0 * RANK + col) = pack_bf16(o[n][0] * inv0, o[n][1] * inv0);
      if (i1 < rows) *reinterpret_cast<uint32_t*>(out + gr1 * RANK + col) = pack_bf16(o[n][2] * inv1, o[n][3] * inv1);
    }
    return;
  }
#pragma unroll
  for (int n = 0; n < VCOLS / 8; ++n) {
    const int col = cs * VCOLS + n * 8 + 2 * tig;
    if (i0 < rows) *reinterpret_cast<float2*>(part_o + (gr0 * splits + split) * RANK + col) = make_float2(o[n][0], o[n][1]);
    if (i1 < rows) *reinterpret_cast<float2*>(part_o + (gr1 * splits + split) * RANK + col) = make_float2(o[n][2], o[n][3]);
  }
  if (cs == 0 && tig == 0) {
    if (i0 < rows) *reinterpret_cast<float2*>(part_ml + (gr0 * splits + split) * 2) = make_float2(m0, l0);
    if (i1 < rows) *reinterpret_cast<float2*>(part_ml + (gr1 * splits + split) * 2) = make_float2(m1, l1);
  }
}

// One block per query row: the splits' sums brought to a common maximum and added in split order.
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
                    int splits, const float* __restrict__ sink_v, int H) {
  const size_t row = blockIdx.x;
  const float* ml = part_ml + row * splits * 2;
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, ml[2 * s]);
  float den = 0.f;
  for (int s = 0; s < splits; ++s)
    if (ml[2 * s] != -INFINITY) den += ml[2 * s + 1] * fast_exp2(ml[2 * s] - mx);
  if (sink_v != nullptr && mx != -INFINITY) den += fast_exp2(sink_v[row % H] * 1.4426950408889634f - mx);
  const float inv = den > 0.f ? 1.0f / den : 0.f;
  for (int c = threadIdx.x; c < RANK; c += blockDim.x) {
    float num = 0.f;
    for (int s = 0; s < splits; ++s)
      if (ml[2 * s] != -INFINITY) num += part_o[(row * splits + s) * RANK + c] * fast_exp2(ml[2 * s] - mx);
    out[row * RANK + c] = __float2bfloat16_rn(num * inv);
  }
}

gb::OncePerDevice smem_set;

}  // namespace

GB_EXPORT int gb_latent_attention_rank() { return RANK; }
GB_EXPORT int gb_latent_attention_rot() { return ROT; }

// Bytes of work space for a launch with `splits` > 1 over `rows` = tokens * heads query rows.
GB_EXPORT long long gb_latent_attention_scratch_bytes(long long rows, int splits) {
  return splits > 1 ? rows * splits * (RANK + 2) * (long long)sizeof(float) : 0;
}

// q [T, H, ROW], pool [pages, 1, page_size, ROW], out [T, H * RANK], all bfloat16. max_q_len: the most
// tokens a request brings (the grid's extent). splits: CTAs that share a tile's keys (1: none).
// sink_v ([H] 32-bit, or null): exp(sink_v[h]) joins head h's softmax denominator.
GB_EXPORT int gb_latent_attention(const void* q, const void* pool, void* out, const int32_t* block_table,
                                  int table_width, const int32_t* cu_q, const int32_t* kv_lens, int T,
                                  int num_requests, int H, float scale, int page_size, int max_q_len, int splits,
                                  void* scratch, long long scratch_bytes, const float* sink_v, cudaStream_t stream) {
  if (T <= 0 || num_requests <= 0) return GB_OK;
  if (H < 1 || page_size < 1 || max_q_len < 1 || splits < 1 || !(scale > 0.f))
    return gb::fail(GB_BAD_ARGUMENT, "latent_attention: heads %d, page size %d, scale %g", H, page_size, (double)scale);
  const long long rows = (long long)T * H;
  if (splits > 1 && (scratch == nullptr || scratch_bytes < gb_latent_attention_scratch_bytes(rows, splits)))
    return gb::fail(GB_BAD_ARGUMENT, "latent_attention: %d splits need %lld bytes of work space", splits,
                    gb_latent_attention_scratch_bytes(rows, splits));
  if (smem_set.needed()) {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e != cudaSuccess) return gb::fail(GB_CUDA_ERROR, "latent_attention: %s", cudaGetErrorString(e));
    smem_set.done();
  }
  float* part_o = (float*)scratch;
  float* part_ml = part_o ? part_o + rows * splits * RANK : nullptr;
  const int tiles = (int)(((long long)max_q_len * H + BM - 1) / BM);
  dim3 grid(tiles, num_requests, splits);
  latent_attention_kernel<<<grid, THREADS, SMEM, stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)pool, (__nv_bfloat16*)out, part_o, part_ml, block_table,
      table_width, cu_q, kv_lens, H, scale * 1.4426950408889634f, page_size, splits, sink_v);
  int rc = gb::check_launch("latent_attention");
  if (rc != GB_OK || splits == 1) return rc;
  latent_merge_kernel<<<(unsigned)rows, 128, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)out, splits, sink_v, H);
  return gb::check_launch("latent_merge");
}
