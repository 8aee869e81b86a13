// Attention over a cached low-rank latent: what lies around the attention kernel itself.
//
// A token caches one vector c = rms(W_dkv h) * g of `rank` elements; head i's keys and values are
// k = Uk_i c and v = Uv_i c.  Nothing but c is stored: the score q_i . k = (Uk_i^T q_i) . c, and the
// weighted sum of values is Uv_i (sum_j p_j c_j), so the attention kernels run with one shared
// "kv head" whose keys and values are both the cached latents, on queries mapped by Uk^T, and
// their output is mapped by Uv afterwards.
//
//   latent_write   c = x / sqrt(mean(x^2) + eps) * g in 32-bit from the projection's columns, stored
//                  into the token's place of its page (dummy rows and released pages are skipped)
//
// A layer may keep a ROTATED KEY PART beside the latent: `tail` more columns of the projection, shared by all
// heads, turned by the token's position in pairs of neighbours (the first `rot` of them; the rest pass) and stored
// behind the latent in the same cache row (row = rank + tail).  Every head's query then ends in `tail` columns of
// its own that are turned the same way and copied behind the head's mapped query, so that one dot product over
// rank + tail elements gives q_a . k_a + q_r . k_r.  The same launch does both; a layer that reads another layer's
// cache runs it for its queries alone (cache null).
//   head_matmul    out[t, i, :] = x[t, i, :] W[i] for every head i, W [heads, K, N]: the two maps
//                  above, 16 tokens a block so that a head's matrix is read once per 16 tokens;
//                  32-bit sums (a step of at most 16 tokens cuts k in four parts that are added in order)
#include <math.h>
#include "common.cuh"
#include "sm100.cuh"

using namespace ilb;

struct LatentWrite {
  const float* w; float eps;
  const int* positions; const int* seq_of_token; const int* block_table;
  int col0, rank, max_blocks, page_size, num_pages;
  // the rotated part (tail 0: none): cos/sin per token [tokens][rot / 2][2]
  int tail, rot;
  const float* angles;
};

// The queries' tails of token t: head i's columns [qcol0 + i * qhs, + tail) of `qsrc` turned into columns
// [rank + i * (rank + tail), + tail) of `qdst`.
struct QueryTails {
  const void* src; void* dst;
  int ld_src, ld_dst, heads, col0, head_stride;
};

template <typename T>
__device__ __forceinline__ void turn_pair(const T* __restrict__ src, int i, int tail, int rot, const float* __restrict__ cs,
                                          float& a, float& b) {
  // elements 2i and 2i + 1 (b unused when 2i + 1 == tail)
  const float u = to_float(src[2 * i]);
  const float v = 2 * i + 1 < tail ? to_float(src[2 * i + 1]) : 0.f;
  if (2 * i + 1 < rot) {
    const float c = cs[2 * i], s = cs[2 * i + 1];
    a = u * c - v * s;
    b = v * c + u * s;
  } else {
    a = u; b = v;
  }
}

// One block of 128 threads writes the latent (and the rotated part) of token t, and turns its queries' tails.
template <typename TI, typename TC, typename TQ = TI>
__device__ __forceinline__ void latent_write_token(const TI* __restrict__ proj, int ld, const LatentWrite& a, TC* __restrict__ cache,
                                                   int t, float* scratch, const QueryTails* qt = nullptr) {
  const int col0 = a.col0, rank = a.rank, max_blocks = a.max_blocks, page_size = a.page_size, num_pages = a.num_pages;
  const int tail = a.tail, rot = a.rot, pairs = (tail + 1) / 2;
  const float* cs = a.angles != nullptr ? a.angles + (size_t)t * rot : nullptr;
  if (qt != nullptr && tail > 0) {
    const TQ* qsrc = reinterpret_cast<const TQ*>(qt->src) + (size_t)t * qt->ld_src + qt->col0;
    TQ* qdst = reinterpret_cast<TQ*>(qt->dst) + (size_t)t * qt->ld_dst + rank;
    for (int e = threadIdx.x; e < qt->heads * pairs; e += blockDim.x) {
      const int h = e / pairs, i = e % pairs;
      float u, v;
      turn_pair<TQ>(qsrc + (size_t)h * qt->head_stride, i, tail, rot, cs, u, v);
      TQ* o = qdst + (size_t)h * (rank + tail);
      o[2 * i] = from_float<TQ>(u);
      if (2 * i + 1 < tail) o[2 * i + 1] = from_float<TQ>(v);
    }
  }
  if (cache == nullptr) return;
  const float* w = a.w;
  const float eps = a.eps;
  const int* positions = a.positions;
  const int* seq_of_token = a.seq_of_token;
  const int* block_table = a.block_table;
  const TI* row = proj + (size_t)t * ld + col0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_float(row[i]);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
  const int pos = positions[t];
  const int page = block_table[(size_t)seq_of_token[t] * max_blocks + pos / page_size];
  if (page < 0 || page >= num_pages) return;
  TC* dst = cache + ((size_t)page * page_size + pos % page_size) * (rank + tail);
  for (int i = threadIdx.x; i < rank; i += blockDim.x)
    dst[i] = from_float<TC>(to_float(row[i]) * inv * w[i]);
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    float u, v;
    turn_pair<TI>(row + rank, i, tail, rot, cs, u, v);
    dst[rank + 2 * i] = from_float<TC>(u);
    if (2 * i + 1 < tail) dst[rank + 2 * i + 1] = from_float<TC>(v);
  }
}

template <typename TI, typename TC>
__global__ void __launch_bounds__(128)
latent_write_kernel(const TI* __restrict__ proj, int ld, const LatentWrite a, TC* __restrict__ cache) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  __shared__ float scratch[33];
  latent_write_token<TI, TC>(proj, ld, a, cache, blockIdx.x, scratch);
}

ILB_EXPORT int ilb_latent_write(const void* proj, int dtype, int ld, int col0, int rank, const float* w, float eps,
                                const int* positions, const int* seq_of_token, const int* block_table, int max_blocks,
                                int page_size, int num_pages, void* cache, int cache_dtype, int n_tokens, cudaStream_t stream) {
  ILB_REQUIRE(rank > 0 && ld >= col0 + rank && n_tokens >= 0 && eps > 0.f, "latent_write: bad sizes");
  ILB_REQUIRE(page_size > 0 && max_blocks > 0 && num_pages > 0, "latent_write: bad cache geometry");
  if (n_tokens == 0) return 0;
  const LatentWrite a{w, eps, positions, seq_of_token, block_table, col0, rank, max_blocks, page_size, num_pages, 0, 0, nullptr};
#define ILB_LW(TI, TC) ilb::launch(latent_write_kernel<TI, TC>, dim3(n_tokens), dim3(128), 0, stream, (const TI*)proj, ld, a, (TC*)cache)
  if (dtype == kF32 && cache_dtype == kF32) ILB_LW(float, float);
  else if (dtype == kBF16 && cache_dtype == kBF16) ILB_LW(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == kBF16 && cache_dtype == kF32) ILB_LW(__nv_bfloat16, float);
  else if (dtype == kF32 && cache_dtype == kBF16) ILB_LW(float, __nv_bfloat16);
  else return fail("latent_write: unsupported dtypes %d/%d", dtype, cache_dtype);
#undef ILB_LW
  return check_launch("latent_write");
}

// The latent with a rotated part behind it, and the queries' tails, of every token of a step (see the top).
template <typename TI, typename TC, typename TQ>
__global__ void __launch_bounds__(128)
latent_write_rot_kernel(const TI* __restrict__ proj, int ld, const LatentWrite a, TC* __restrict__ cache, const QueryTails qt) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  __shared__ float scratch[33];
  latent_write_token<TI, TC, TQ>(proj, ld, a, cache, blockIdx.x, scratch, qt.src != nullptr ? &qt : nullptr);
}

// proj [T, ld] (`dtype`): the latent's columns from col0, the part to rotate right behind them; cache rows of
// rank + tail elements (null: nothing is stored); angles [T, rot / 2, 2] (cos, sin); q_src [T, ld_q] (`q_dtype`), head i's
// tail at columns q_col0 + i * q_head_stride; q_dst [T, heads * (rank + tail)].
ILB_EXPORT int ilb_latent_write_rot(const void* proj, int dtype, int ld, int col0, int rank, int tail, int rot, const float* angles,
                                    const float* w, float eps, const int* positions, const int* seq_of_token, const int* block_table,
                                    int max_blocks, int page_size, int num_pages, void* cache, int cache_dtype, const void* q_src,
                                    void* q_dst, int q_dtype, int ld_q, int q_col0, int q_head_stride, int heads, int n_tokens,
                                    cudaStream_t stream) {
  ILB_REQUIRE(rank > 0 && tail >= 0 && n_tokens >= 0, "latent_write_rot: bad sizes");
  ILB_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= tail && (rot == 0 || angles != nullptr), "latent_write_rot: %d of %d elements cannot turn in pairs", rot, tail);
  ILB_REQUIRE(cache == nullptr || (ld >= col0 + rank + tail && eps > 0.f && w != nullptr && page_size > 0 && max_blocks > 0 && num_pages > 0),
              "latent_write_rot: bad cache geometry");
  ILB_REQUIRE(q_src == nullptr || (q_dst != nullptr && heads > 0 && q_head_stride >= tail && ld_q >= q_col0 + (heads - 1) * q_head_stride + tail),
              "latent_write_rot: the queries' rows are too short");
  ILB_REQUIRE(cache != nullptr || q_src != nullptr, "latent_write_rot: nothing to do");
  if (n_tokens == 0) return 0;
  const LatentWrite a{w, eps, positions, seq_of_token, block_table, col0, rank, max_blocks, page_size, num_pages, tail, rot, angles};
  const QueryTails qt{q_src, q_dst, ld_q, heads * (rank + tail), heads, q_col0, q_head_stride};
#define ILB_LW(TI, TC, TQ) ilb::launch(latent_write_rot_kernel<TI, TC, TQ>, dim3(n_tokens), dim3(128), 0, stream, (const TI*)proj, ld, a, (TC*)cache, qt)
  const int cd = cache != nullptr ? cache_dtype : q_dtype;
  if (dtype == kF32 && cd == kF32 && q_dtype == kF32) ILB_LW(float, float, float);
  else if (dtype == kF32 && cd == kBF16 && q_dtype == kBF16) ILB_LW(float, __nv_bfloat16, __nv_bfloat16);
  else if (dtype == kBF16 && cd == kBF16 && q_dtype == kBF16) ILB_LW(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  else return fail("latent_write_rot: unsupported dtypes %d/%d/%d", dtype, cd, q_dtype);
#undef ILB_LW
  return check_launch("latent_write_rot");
}

constexpr int kHeadTokens = 16;

// Block (128 / KS columns n) x (KS ranges of k).  Many tokens: KS = 1, a thread owns a column for 16 tokens.  A step
// of few tokens has few blocks of that kind, so its k range is cut in four and the parts meet in shared memory.
template <typename TI, typename TW, typename TO, int KS>
__device__ __forceinline__ void head_matmul_block(const TI* __restrict__ x, int ldx, const TW* __restrict__ w, TO* __restrict__ out,
                                                  int ldo, int n_tokens, int K, int N, int xhs, int ohs, int t0, int h, int n_block, float* xs) {
  constexpr int NT = 128 / KS;
  const int ts = min(kHeadTokens, n_tokens - t0);
  for (int i = threadIdx.x; i < kHeadTokens * K; i += 128) {
    const int tt = i / K, k = i % K;
    xs[i] = tt < ts ? to_float(x[(size_t)(t0 + tt) * ldx + (size_t)h * xhs + k]) : 0.f;
  }
  __syncthreads();
  const int tn = threadIdx.x % NT, tk = threadIdx.x / NT;
  const int n = n_block * NT + tn;
  const bool live = n < N;
  const int per = ((K + KS - 1) / KS + 3) / 4 * 4;
  const int k0 = tk * per, k1 = min(K, k0 + per);
  float acc[kHeadTokens];
#pragma unroll
  for (int tt = 0; tt < kHeadTokens; ++tt) acc[tt] = 0.f;
  const TW* wp = w + (size_t)h * K * N + (live ? n : 0);
  int k = k0;
  if (K % 4 == 0) {
    for (; k + 4 <= k1; k += 4) {
      const float w0 = to_float(wp[(size_t)k * N]), w1 = to_float(wp[(size_t)(k + 1) * N]);
      const float w2 = to_float(wp[(size_t)(k + 2) * N]), w3 = to_float(wp[(size_t)(k + 3) * N]);
#pragma unroll
      for (int tt = 0; tt < kHeadTokens; ++tt) {
        const float4 v = *reinterpret_cast<const float4*>(xs + tt * K + k);
        acc[tt] = fmaf(v.x, w0, acc[tt]); acc[tt] = fmaf(v.y, w1, acc[tt]);
        acc[tt] = fmaf(v.z, w2, acc[tt]); acc[tt] = fmaf(v.w, w3, acc[tt]);
      }
    }
  }
  for (; k < k1; ++k) {
    const float wv = to_float(wp[(size_t)k * N]);
#pragma unroll
    for (int tt = 0; tt < kHeadTokens; ++tt) acc[tt] = fmaf(xs[tt * K + k], wv, acc[tt]);
  }
  if (KS > 1) {
    float* red = xs + kHeadTokens * K;
#pragma unroll
    for (int tt = 0; tt < kHeadTokens; ++tt) red[(tk * kHeadTokens + tt) * NT + tn] = acc[tt];
    __syncthreads();
    if (tk != 0) return;
#pragma unroll
    for (int tt = 0; tt < kHeadTokens; ++tt) {
      float v = 0.f;
      for (int r = 0; r < KS; ++r) v += red[(r * kHeadTokens + tt) * NT + tn];
      acc[tt] = v;
    }
  }
  if (!live) return;
#pragma unroll
  for (int tt = 0; tt < kHeadTokens; ++tt)
    if (tt < ts) out[(size_t)(t0 + tt) * ldo + (size_t)h * ohs + n] = from_float<TO>(acc[tt]);
}

template <typename TI, typename TW, typename TO, int KS>
__global__ void __launch_bounds__(128)
head_matmul_kernel(const TI* __restrict__ x, int ldx, const TW* __restrict__ w, TO* __restrict__ out, int ldo,
                   int n_tokens, int K, int N, int xhs, int ohs) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  extern __shared__ __align__(16) float xs[];           // [kHeadTokens][K], then (KS > 1) [KS][kHeadTokens][NT]
  head_matmul_block<TI, TW, TO, KS>(x, ldx, w, out, ldo, n_tokens, K, N, xhs, ohs, blockIdx.x * kHeadTokens, blockIdx.y, blockIdx.z, xs);
}

// The input stage of a step of few tokens in one launch: blocks (tile of 16 tokens, head, 32 columns) map the queries
// to the latent space, and sixteen more blocks a tile write the latents of its tokens.
template <typename TI, typename TC, typename TO>
__global__ void __launch_bounds__(128)
latent_input_kernel(const TI* __restrict__ proj, int ld, const TI* __restrict__ w, TO* __restrict__ q_out, int ldo, int n_tokens,
                    int heads, int K, int N, const LatentWrite a, TC* __restrict__ cache) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  extern __shared__ __align__(16) float xs[];
  __shared__ float scratch[33];
  const int n_blocks = (N + 31) / 32, t0 = blockIdx.x * kHeadTokens;
  const int y = blockIdx.y;
  if (y < heads * n_blocks) {
    head_matmul_block<TI, TI, TO, 4>(proj, ld, w, q_out, ldo, n_tokens, K, N, K, N, t0, y / n_blocks, y % n_blocks, xs);
  } else {
    const int t = t0 + (y - heads * n_blocks);
    if (t < n_tokens) latent_write_token<TI, TC>(proj, ld, a, cache, t, scratch);
  }
}

// The same product for many bfloat16 tokens on the tensor cores (mma.sync m16n8k16, 32-bit sums): a block of four
// warps takes 64 tokens x 64 columns of one head; the head's matrix passes through shared memory in slices of 64 k
// ([k][n] as stored, read with ldmatrix.trans), the tokens' rows come straight from global memory as A fragments.
// K a multiple of 16, N of 8.
constexpr int kMmaTile = 64;

__global__ void __launch_bounds__(128)
head_matmul_mma_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ w,
                       __nv_bfloat16* __restrict__ out, int ldo, int n_tokens, int K, int N, int xhs, int ohs) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  __shared__ __align__(16) __nv_bfloat16 ws[kMmaTile][kMmaTile + 8];
  const int t0 = blockIdx.x * kMmaTile, h = blockIdx.y, n0 = blockIdx.z * kMmaTile;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int r0 = t0 + warp * 16 + g, r1 = r0 + 8;
  const bool live0 = r0 < n_tokens, live1 = r1 < n_tokens;
  const __nv_bfloat16* a0 = x + (size_t)(live0 ? r0 : 0) * ldx + (size_t)h * xhs;
  const __nv_bfloat16* a1 = x + (size_t)(live1 ? r1 : 0) * ldx + (size_t)h * xhs;
  float acc[kMmaTile / 8][4];
#pragma unroll
  for (int i = 0; i < kMmaTile / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
  for (int k0 = 0; k0 < K; k0 += kMmaTile) {
    __syncthreads();
#pragma unroll
    for (int it = 0; it < kMmaTile * (kMmaTile / 8) / 128; ++it) {
      const int idx = threadIdx.x + it * 128, r = idx / (kMmaTile / 8), cv = idx % (kMmaTile / 8);
      const int k = k0 + r, n = n0 + cv * 8;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (k < K && n < N) v = __ldg(reinterpret_cast<const uint4*>(w + ((size_t)h * K + k) * N + n));
      *reinterpret_cast<uint4*>(&ws[r][cv * 8]) = v;
    }
    __syncthreads();
#pragma unroll
    for (int kb = 0; kb < kMmaTile / 16; ++kb) {
      const int c = k0 + kb * 16 + 2 * t;
      if (k0 + kb * 16 >= K) break;
      uint32_t a[4];
      a[0] = live0 ? *reinterpret_cast<const uint32_t*>(a0 + c) : 0u;
      a[1] = live1 ? *reinterpret_cast<const uint32_t*>(a1 + c) : 0u;
      a[2] = live0 ? *reinterpret_cast<const uint32_t*>(a0 + c + 8) : 0u;
      a[3] = live1 ? *reinterpret_cast<const uint32_t*>(a1 + c + 8) : 0u;
#pragma unroll
      for (int nd = 0; nd < kMmaTile / 16; ++nd) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(smem_u32(&ws[kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][nd * 16 + (lane >> 4) * 8]), b0, b1, b2, b3);
        mma_16816(acc[2 * nd], a, b0, b1);
        mma_16816(acc[2 * nd + 1], a, b2, b3);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kMmaTile / 8; ++i) {
    const int col = n0 + i * 8 + 2 * t;
    if (col >= N) continue;
    if (live0) *reinterpret_cast<uint32_t*>(out + (size_t)r0 * ldo + (size_t)h * ohs + col) = pack_bf16(acc[i][0], acc[i][1]);
    if (live1) *reinterpret_cast<uint32_t*>(out + (size_t)r1 * ldo + (size_t)h * ohs + col) = pack_bf16(acc[i][2], acc[i][3]);
  }
}

// The same tiles for 32-bit rows times a bfloat16 matrix with a 32-bit result that keeps 32-bit accuracy: every input is
// cut into three bfloat16 pieces (x = hi + mid + lo exactly, 8 + 8 + 8 significant bits), each piece's products with the
// bfloat16 matrix are exact in 32 bits, and the three products are accumulated in 32-bit, the smallest piece first.
__device__ __forceinline__ void split3(float2 v, uint32_t& hi, uint32_t& mid, uint32_t& lo) {
  const __nv_bfloat16 h0 = __float2bfloat16_rn(v.x), h1 = __float2bfloat16_rn(v.y);
  const float r0 = v.x - __bfloat162float(h0), r1 = v.y - __bfloat162float(h1);
  const __nv_bfloat16 m0 = __float2bfloat16_rn(r0), m1 = __float2bfloat16_rn(r1);
  const __nv_bfloat16 l0 = __float2bfloat16_rn(r0 - __bfloat162float(m0)), l1 = __float2bfloat16_rn(r1 - __bfloat162float(m1));
  hi = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
  mid = (uint32_t)__bfloat16_as_ushort(m0) | ((uint32_t)__bfloat16_as_ushort(m1) << 16);
  lo = (uint32_t)__bfloat16_as_ushort(l0) | ((uint32_t)__bfloat16_as_ushort(l1) << 16);
}

__global__ void __launch_bounds__(128)
head_matmul_split_kernel(const float* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ w, float* __restrict__ out, int ldo,
                         int n_tokens, int K, int N, int xhs, int ohs) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  __shared__ __align__(16) __nv_bfloat16 ws[kMmaTile][kMmaTile + 8];
  const int t0 = blockIdx.x * kMmaTile, h = blockIdx.y, n0 = blockIdx.z * kMmaTile;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int r0 = t0 + warp * 16 + g, r1 = r0 + 8;
  const bool live0 = r0 < n_tokens, live1 = r1 < n_tokens;
  const float* a0 = x + (size_t)(live0 ? r0 : 0) * ldx + (size_t)h * xhs;
  const float* a1 = x + (size_t)(live1 ? r1 : 0) * ldx + (size_t)h * xhs;
  const bool warp_live = t0 + warp * 16 < n_tokens;          // (a warp whose 16 rows are all past the end only helps with the copies)
  float acc[kMmaTile / 8][4];
#pragma unroll
  for (int i = 0; i < kMmaTile / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
  for (int k0 = 0; k0 < K; k0 += kMmaTile) {
    __syncthreads();
#pragma unroll
    for (int it = 0; it < kMmaTile * (kMmaTile / 8) / 128; ++it) {
      const int idx = threadIdx.x + it * 128, r = idx / (kMmaTile / 8), cv = idx % (kMmaTile / 8);
      const int k = k0 + r, n = n0 + cv * 8;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (k < K && n < N) v = __ldg(reinterpret_cast<const uint4*>(w + ((size_t)h * K + k) * N + n));
      *reinterpret_cast<uint4*>(&ws[r][cv * 8]) = v;
    }
    __syncthreads();
    if (!warp_live) continue;
#pragma unroll
    for (int kb = 0; kb < kMmaTile / 16; ++kb) {
      const int c = k0 + kb * 16 + 2 * t;
      if (k0 + kb * 16 >= K) break;
      const float2 zero = make_float2(0.f, 0.f);
      uint32_t hi[4], mid[4], lo[4];
      split3(live0 ? *reinterpret_cast<const float2*>(a0 + c) : zero, hi[0], mid[0], lo[0]);
      split3(live1 ? *reinterpret_cast<const float2*>(a1 + c) : zero, hi[1], mid[1], lo[1]);
      split3(live0 ? *reinterpret_cast<const float2*>(a0 + c + 8) : zero, hi[2], mid[2], lo[2]);
      split3(live1 ? *reinterpret_cast<const float2*>(a1 + c + 8) : zero, hi[3], mid[3], lo[3]);
#pragma unroll
      for (int nd = 0; nd < kMmaTile / 16; ++nd) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(smem_u32(&ws[kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][nd * 16 + (lane >> 4) * 8]), b0, b1, b2, b3);
        mma_16816(acc[2 * nd], lo, b0, b1);
        mma_16816(acc[2 * nd + 1], lo, b2, b3);
        mma_16816(acc[2 * nd], mid, b0, b1);
        mma_16816(acc[2 * nd + 1], mid, b2, b3);
        mma_16816(acc[2 * nd], hi, b0, b1);
        mma_16816(acc[2 * nd + 1], hi, b2, b3);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kMmaTile / 8; ++i) {
    const int col = n0 + i * 8 + 2 * t;
    if (col >= N) continue;
    if (live0) *reinterpret_cast<float2*>(out + (size_t)r0 * ldo + (size_t)h * ohs + col) = make_float2(acc[i][0], acc[i][1]);
    if (live1) *reinterpret_cast<float2*>(out + (size_t)r1 * ldo + (size_t)h * ohs + col) = make_float2(acc[i][2], acc[i][3]);
  }
}

// x: [T, ldx] 32-bit, head i at columns i * xhs ..; w: [heads, K, N] bfloat16; out: [T, ldo] 32-bit, head i at columns
// i * ohs ...  K a multiple of 16, N of 8; strides and head offsets even; x and out 8-byte aligned, w 16-byte aligned.
ILB_EXPORT int ilb_head_matmul_split(const float* x, int ldx, const void* w, float* out, int ldo, int n_tokens, int heads, int K, int N,
                                     int xhs, int ohs, cudaStream_t stream) {
  ILB_REQUIRE(n_tokens >= 0 && heads > 0 && heads <= 65535 && K > 0 && N > 0, "head_matmul_split: bad sizes");
  ILB_REQUIRE(xhs >= K && ohs >= N && ldx >= (heads - 1) * xhs + K && ldo >= (heads - 1) * ohs + N, "head_matmul_split: strides too small");
  ILB_REQUIRE(K % 16 == 0 && N % 8 == 0 && ldx % 2 == 0 && ldo % 2 == 0 && xhs % 2 == 0 && ohs % 2 == 0 && ((uintptr_t)x % 8 == 0) &&
              ((uintptr_t)out % 8 == 0) && ((uintptr_t)w % 16 == 0), "head_matmul_split: sizes or alignment not served");
  if (n_tokens == 0) return 0;
  const dim3 grid((n_tokens + kMmaTile - 1) / kMmaTile, heads, (N + kMmaTile - 1) / kMmaTile);
  ILB_REQUIRE(grid.z <= 65535, "head_matmul_split: too many columns");
  ilb::launch(head_matmul_split_kernel, grid, dim3(128), 0, stream, x, ldx, (const __nv_bfloat16*)w, out, ldo, n_tokens, K, N, xhs, ohs);
  return check_launch("head_matmul_split");
}

// x: [T, ldx] of `dtype`, head i at columns i * xhs ..; w: [heads, K, N] of `dtype`; out: [T, ldo] of
// `out_dtype`, head i at columns i * ohs ... (xhs >= K and ohs >= N: a head's row may hold more than the product reads or writes)
ILB_EXPORT int ilb_head_matmul(const void* x, int dtype, int ldx, const void* w, void* out, int out_dtype, int ldo,
                               int n_tokens, int heads, int K, int N, int xhs, int ohs, cudaStream_t stream) {
  ILB_REQUIRE(n_tokens >= 0 && heads > 0 && heads <= 65535 && K > 0 && N > 0, "head_matmul: bad sizes");
  ILB_REQUIRE(xhs >= K && ohs >= N && ldx >= (heads - 1) * xhs + K && ldo >= (heads - 1) * ohs + N, "head_matmul: strides too small");
  if (dtype == kBF16 && out_dtype == kBF16 && n_tokens > kHeadTokens && K % 16 == 0 && N % 8 == 0 && ldx % 2 == 0 && ldo % 2 == 0 &&
      xhs % 2 == 0 && ohs % 2 == 0 &&
      ((uintptr_t)x % 4 == 0) && ((uintptr_t)out % 4 == 0) && ((uintptr_t)w % 16 == 0)) {
    const dim3 grid((n_tokens + kMmaTile - 1) / kMmaTile, heads, (N + kMmaTile - 1) / kMmaTile);
    ilb::launch(head_matmul_mma_kernel, grid, dim3(128), 0, stream, (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w,
                (__nv_bfloat16*)out, ldo, n_tokens, K, N, xhs, ohs);
    return check_launch("head_matmul");
  }
  const bool few = n_tokens <= kHeadTokens;
  const size_t smem = sizeof(float) * kHeadTokens * ((size_t)K + (few ? 128 : 0));
  ILB_REQUIRE(smem <= 48 * 1024, "head_matmul: inner size %d exceeds %d", K, 48 * 1024 / 4 / kHeadTokens - 128);
  if (n_tokens == 0) return 0;
  const int nt = few ? 32 : 128;
  const dim3 grid((n_tokens + kHeadTokens - 1) / kHeadTokens, heads, (N + nt - 1) / nt);
#define ILB_HM(TI, TO)                                                                                                        \
  do {                                                                                                                        \
    if (few) ilb::launch(head_matmul_kernel<TI, TI, TO, 4>, grid, dim3(128), smem, stream, (const TI*)x, ldx, (const TI*)w,   \
                         (TO*)out, ldo, n_tokens, K, N, xhs, ohs);                                                            \
    else ilb::launch(head_matmul_kernel<TI, TI, TO, 1>, grid, dim3(128), smem, stream, (const TI*)x, ldx, (const TI*)w,       \
                     (TO*)out, ldo, n_tokens, K, N, xhs, ohs);                                                                \
  } while (0)
  if (dtype == kF32 && out_dtype == kF32) ILB_HM(float, float);
  else if (dtype == kBF16 && out_dtype == kBF16) ILB_HM(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == kBF16 && out_dtype == kF32) ILB_HM(__nv_bfloat16, float);
  else return fail("head_matmul: unsupported dtypes %d/%d", dtype, out_dtype);
#undef ILB_HM
  return check_launch("head_matmul");
}

// ilb_latent_write and ilb_head_matmul (queries: heads x K at the row's start) of a step of few tokens as one launch.
ILB_EXPORT int ilb_latent_input(const void* proj, int dtype, int ld, const void* w, void* q_out, int out_dtype, int ldo, int n_tokens,
                                int heads, int K, int N, int col0, int rank, const float* norm_w, float eps, const int* positions,
                                const int* seq_of_token, const int* block_table, int max_blocks, int page_size, int num_pages,
                                void* cache, int cache_dtype, cudaStream_t stream) {
  ILB_REQUIRE(n_tokens >= 0 && heads > 0 && K > 0 && N > 0 && rank > 0 && eps > 0.f, "latent_input: bad sizes");
  ILB_REQUIRE(ld >= heads * K && ld >= col0 + rank && ldo >= heads * N, "latent_input: strides too small");
  ILB_REQUIRE(page_size > 0 && max_blocks > 0 && num_pages > 0, "latent_input: bad cache geometry");
  const size_t smem = sizeof(float) * kHeadTokens * ((size_t)K + 128);
  ILB_REQUIRE(smem <= 48 * 1024, "latent_input: inner size %d exceeds %d", K, 48 * 1024 / 4 / kHeadTokens - 128);
  const long long rows = (long long)heads * ((N + 31) / 32) + kHeadTokens;
  ILB_REQUIRE(rows <= 65535, "latent_input: too many heads");
  if (n_tokens == 0) return 0;
  const LatentWrite a{norm_w, eps, positions, seq_of_token, block_table, col0, rank, max_blocks, page_size, num_pages, 0, 0, nullptr};
  const dim3 grid((n_tokens + kHeadTokens - 1) / kHeadTokens, (unsigned)rows);
#define ILB_LI(TI, TC, TO) ilb::launch(latent_input_kernel<TI, TC, TO>, grid, dim3(128), smem, stream, (const TI*)proj, ld, (const TI*)w, \
                                        (TO*)q_out, ldo, n_tokens, heads, K, N, a, (TC*)cache)
  if (dtype == kF32 && cache_dtype == kF32 && out_dtype == kF32) ILB_LI(float, float, float);
  else if (dtype == kBF16 && cache_dtype == kBF16 && out_dtype == kBF16) ILB_LI(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  else return fail("latent_input: unsupported dtypes %d/%d/%d", dtype, cache_dtype, out_dtype);
#undef ILB_LI
  return check_launch("latent_input");
}

ILB_DEFINE_LAST_ERROR()
