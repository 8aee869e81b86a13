// Causal grouped-query attention whose scores are reshaped and MIXED ACROSS HEADS before the softmax,
// over the paged cache, any batch shape, exact 32-bit.
//
// For the token at position i of a sequence, key j <= i (j >= i - window + 1 with a window), query head g:
//
//     s_g  = scale * temp(i) * q_g . k_j            temp(i) = 1 + coef * ln(floor((i + 1) / every) + 1)   (coef 0: 1)
//     s_g <- cap * tanh(s_g / cap)                   (cap 0: left as it is)
//     s_g <- s_g - r1_g * ln(1 + r2_g * (i - j))     (r1 null: no distance term)
//     z_h  = sum_g M[h, g] * s_g                     (M null: z = s)
//     p_h  = exp(z_h) / (exp(sink_h) + sum_j exp(z_h))          (sink null: the plain softmax)
//     o_h  = sum_j p_h v_j,  v of kv head h / (nq / nkv)
//
// Because every head's probabilities need every head's scores, one block owns a token with ALL its heads.
// It walks the keys in tiles of 32 in the order of their positions: scores (a warp a head, a lane a key),
// mixing and the running softmax (a warp a head), then the weighted values (a thread an output element).
// The walk depends on the token's position alone, so a result never depends on the batch or on how the
// tokens were cut into steps.  Keys and queries have head size d, values dv.
#include <math.h>
#include "common.cuh"

using namespace ilb;

constexpr int kMixThreads = 256;
constexpr int kMixWarps = kMixThreads / 32;
constexpr int kMixTile = 32;
constexpr int kMixAcc = 32;            // output elements a thread may own: nq * dv <= 256 * 32

struct MixParams {
  const int* positions; const int* seq_of_token; const int* block_table;
  int max_blocks, page_size, num_pages, window;
  float scale;
  int nq, nkv, d, dv, q_stride, out_stride;
  const float* sink; const float* talk; const float* r1; const float* r2;
  float softcap, temp_coef;
  int temp_every;
};

template <typename TQ, typename TC>
__global__ void __launch_bounds__(kMixThreads)
attention_mix_kernel(const TQ* __restrict__ q, TQ* __restrict__ out, const TC* __restrict__ k_cache,
                     const TC* __restrict__ v_cache, const MixParams a) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  extern __shared__ __align__(16) float sm[];
  const int nq = a.nq, nkv = a.nkv, d = a.d, dv = a.dv;
  float* qs = sm;                              // [nq][d]
  float* S = qs + (size_t)nq * d;              // [nq][32] shaped scores
  float* P = S + nq * kMixTile;                // [nq][32] weights of the tile
  float* m_s = P + nq * kMixTile;              // [nq] running maximum
  float* l_s = m_s + nq;                       // [nq] running sum
  float* c_s = l_s + nq;                       // [nq] what the tile scales the old sums by
  int* row_s = reinterpret_cast<int*>(c_s + nq);   // [32] page * page_size + place of the tile's keys, -1: not read
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per = nq / nkv;
  const int p = a.positions[t];
  const int lo = (a.window > 0 && p + 1 > a.window) ? p + 1 - a.window : 0;
  const int* table = a.block_table + (size_t)a.seq_of_token[t] * a.max_blocks;
  float temp = 1.0f;
  if (a.temp_coef != 0.f) temp = 1.0f + a.temp_coef * logf((float)((p + 1) / a.temp_every) + 1.0f);
  const float qscale = a.scale * temp;

  for (int i = threadIdx.x; i < nq * d; i += kMixThreads)
    qs[i] = to_float(q[(size_t)t * a.q_stride + i]);
  for (int h = threadIdx.x; h < nq; h += kMixThreads) { m_s[h] = -INFINITY; l_s[h] = 0.f; }
  float acc[kMixAcc];
#pragma unroll
  for (int i = 0; i < kMixAcc; ++i) acc[i] = 0.f;
  __syncthreads();

  const int n_tiles = (p - lo + kMixTile) / kMixTile;
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int j0 = lo + tile * kMixTile;
    if (warp == 0) {
      const int j = j0 + lane;
      int row = -1;
      if (j <= p) {
        const int page = table[j / a.page_size];
        if (page >= 0 && page < a.num_pages) row = page * a.page_size + j % a.page_size;
      }
      row_s[lane] = row;
    }
    __syncthreads();
    // scores of every head against the tile's keys, shaped
    {
      const int row = row_s[lane];
      const float dist = (float)(p - (j0 + lane));
      for (int g = warp; g < nq; g += kMixWarps) {
        float s = 0.f;
        if (row >= 0) {
          const int page = row / a.page_size, place = row % a.page_size;
          const TC* kr = k_cache + (((size_t)page * nkv + g / per) * a.page_size + place) * d;
          const float* qg = qs + (size_t)g * d;
          float dot = 0.f;
          for (int i = 0; i < d; ++i) dot = fmaf(qg[i], to_float(kr[i]), dot);
          s = dot * qscale;
          if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
          if (a.r1 != nullptr) s -= a.r1[g] * log1pf(a.r2[g] * dist);
        }
        S[g * kMixTile + lane] = s;
      }
    }
    __syncthreads();
    // mixing across heads, then the running softmax of each head
    {
      const bool seen = row_s[lane] >= 0;
      for (int h = warp; h < nq; h += kMixWarps) {
        float z;
        if (a.talk != nullptr) {
          z = 0.f;
          const float* mh = a.talk + (size_t)h * nq;
          for (int g = 0; g < nq; ++g) z = fmaf(mh[g], S[g * kMixTile + lane], z);
        } else {
          z = S[h * kMixTile + lane];
        }
        if (!seen) z = -INFINITY;
        const float m_old = m_s[h], l_old = l_s[h];
        const float m_new = fmaxf(m_old, warp_max(z));
        const float w = (z == -INFINITY) ? 0.f : expf(z - m_new);
        const float corr = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
        const float sum = warp_sum(w);
        P[h * kMixTile + lane] = w;
        __syncwarp();
        if (lane == 0) { m_s[h] = m_new; l_s[h] = l_old * corr + sum; c_s[h] = corr; }
      }
    }
    __syncthreads();
    // weighted values
#pragma unroll
    for (int r = 0; r < kMixAcc; ++r) {
      const int e = threadIdx.x + r * kMixThreads;
      if (e >= nq * dv) break;
      const int h = e / dv, c = e % dv;
      float v = acc[r] * c_s[h];
      const float* ph = P + h * kMixTile;
      const int kvh = h / per;
      for (int jj = 0; jj < kMixTile; ++jj) {
        const int row = row_s[jj];
        if (row < 0) continue;
        const int page = row / a.page_size, place = row % a.page_size;
        v = fmaf(ph[jj], to_float(v_cache[(((size_t)page * nkv + kvh) * a.page_size + place) * dv + c]), v);
      }
      acc[r] = v;
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < kMixAcc; ++r) {
    const int e = threadIdx.x + r * kMixThreads;
    if (e >= nq * dv) break;
    const int h = e / dv;
    float m = m_s[h], l = l_s[h], f = 1.0f;
    if (a.sink != nullptr) {
      const float top = fmaxf(m, a.sink[h]);
      f = (m == -INFINITY) ? 0.f : expf(m - top);
      l = l * f + expf(a.sink[h] - top);
    }
    out[(size_t)t * a.out_stride + e] = from_float<TQ>(l > 0.f ? acc[r] * f / l : 0.f);
  }
}

ILB_EXPORT int ilb_attention_mix(
    const void* q, void* out, int dtype, const void* k_cache, const void* v_cache, int cache_dtype,
    const int* positions, const int* seq_of_token, const int* block_table, int max_blocks,
    int page_size, int num_pages, int window, float scale, int n_tokens, int nq, int nkv, int d, int dv,
    int q_stride, int out_stride, const float* sink, const float* talk, const float* r1, const float* r2,
    float softcap, float temp_coef, int temp_every, cudaStream_t stream) {
  ILB_REQUIRE(n_tokens >= 0 && nq > 0 && nkv > 0 && d > 0 && dv > 0, "attention_mix: bad sizes");
  ILB_REQUIRE(nq % nkv == 0, "attention_mix: %d query heads are not a multiple of %d kv heads", nq, nkv);
  ILB_REQUIRE((long long)nq * dv <= (long long)kMixThreads * kMixAcc, "attention_mix: %d heads of %d values exceed %d outputs a token",
              nq, dv, kMixThreads * kMixAcc);
  ILB_REQUIRE(page_size > 0 && max_blocks > 0 && num_pages > 0, "attention_mix: bad cache geometry");
  ILB_REQUIRE(window >= 0 && softcap >= 0.f, "attention_mix: negative window or cap");
  ILB_REQUIRE((r1 == nullptr) == (r2 == nullptr), "attention_mix: the distance term needs both of its vectors");
  ILB_REQUIRE(temp_coef == 0.f || temp_every > 0, "attention_mix: the query temperature needs a positive period");
  ILB_REQUIRE(q_stride >= nq * d && out_stride >= nq * dv, "attention_mix: strides too small");
  const size_t smem = sizeof(float) * ((size_t)nq * d + 2 * (size_t)nq * kMixTile + 3 * (size_t)nq) + sizeof(int) * kMixTile;
  ILB_REQUIRE(smem <= 200 * 1024, "attention_mix: %d heads of %d do not fit the block's shared memory", nq, d);
  if (n_tokens == 0) return 0;
  const MixParams a{positions, seq_of_token, block_table, max_blocks, page_size, num_pages, window, scale, nq, nkv, d, dv,
                    q_stride, out_stride, sink, talk, r1, r2, softcap, temp_coef, temp_every};
#define ILB_LAUNCH(TQ, TC)                                                                                              \
  do {                                                                                                                  \
    static OncePerDevice once;                                                                                          \
    if (once.first() && cudaFuncSetAttribute(attention_mix_kernel<TQ, TC>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                             200 * 1024) != cudaSuccess) {                                              \
      once.forget();                                                                                                    \
      return fail("attention_mix: cannot set the shared memory size: %s", cudaGetErrorString(cudaGetLastError()));      \
    }                                                                                                                   \
    ilb::launch(attention_mix_kernel<TQ, TC>, dim3(n_tokens), dim3(kMixThreads), smem, stream, (const TQ*)q, (TQ*)out,  \
                (const TC*)k_cache, (const TC*)v_cache, a);                                                             \
  } while (0)
  if (dtype == kF32 && cache_dtype == kF32) ILB_LAUNCH(float, float);
  else if (dtype == kBF16 && cache_dtype == kBF16) ILB_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else return fail("attention_mix: unsupported dtypes %d/%d", dtype, cache_dtype);
#undef ILB_LAUNCH
  return check_launch("attention_mix");
}

ILB_DEFINE_LAST_ERROR()
