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

// ---------------------------------------------------------------------------------------------------------------
// The same attention on the tensor cores, for a bfloat16 cache (mma.sync m16n8k16, 32-bit sums).
//
// A block of 16 warps owns 16 consecutive tokens of one sequence with ALL heads (at most 16: a warp a head) and
// walks the keys in tiles of 32.  Per tile: the keys and values of every kv head land in shared memory once
// (cp.async); warp g forms head g's 16 x 32 scores, shapes them in 32-bit (temperature, cap, distance term) and
// leaves them in shared memory; after a barrier warp h mixes its head's scores out of all heads' (32-bit multiply-
// adds, the matrix row from shared memory), runs the online softmax on them in registers and multiplies the
// probabilities (rounded to bfloat16, as the engine's other tensor-core attention does) into head h's values.
// The mixed scores have the accumulator layout of the first product, which is the A-operand layout of the second.
//
// A step of single tokens cuts every sequence's keys into chunks of `split_chunk` keys (boundaries by key index
// alone): block (sequence, chunk) leaves (max, sum, weighted values) of its chunk in a scratch record and a
// second launch adds the records in chunk order, with the sink.  Head sizes in multiples of 16, keys up to 128
// (256 with few heads), values up to 128.
#include "sm100.cuh"

constexpr int kTcThreads = 512;
constexpr int kTcWarps = kTcThreads / 32;
constexpr int kTcRows = 16;
constexpr int kTcKeys = 32;
constexpr int kTcSStride = 40;                 // floats between two rows of a head's score tile

struct MixTcParams {
  const __nv_bfloat16* q; __nv_bfloat16* out; const __nv_bfloat16* k_cache; const __nv_bfloat16* v_cache;
  const int* positions; const int* cu_q; const int* block_table;
  int max_blocks, page_size, num_pages, window;
  float scale;
  int n_seqs, nq, nkv, d, dv, q_stride, out_stride;
  const float* sink; const float* talk; const float* r1; const float* r2;
  float softcap, temp_coef;
  int temp_every;
  int split_chunk, max_chunks;
  float* scratch;                              // [n_seqs][max_chunks][nq][dv + 2]
};

__device__ __forceinline__ void mix_cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void mix_cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// tanh and ln(1 + x) from the fast exponential and logarithm: errors of a few 1e-7, far inside bfloat16's.
__device__ __forceinline__ float fast_tanh(float x) {
  const float e = __expf(2.0f * fminf(fmaxf(x, -15.f), 15.f));
  return __fdividef(e - 1.0f, e + 1.0f);
}

template <int DV>
__global__ void __launch_bounds__(kTcThreads, 1)
attention_mix_tc_kernel(const MixTcParams a) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = a.nq, G = a.nkv, d = a.d, dv = a.dv, per = H / G;
  const int qs = d + 8, vs = dv + 8;                                   // row strides (elements) of Q / K and of V
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [H][16][qs]
  __nv_bfloat16* Ks = Qs + (size_t)H * kTcRows * qs;                   // [G][32][qs]
  __nv_bfloat16* Vs = Ks + (size_t)G * kTcKeys * qs;                   // [G][32][vs]
  float* Ss = reinterpret_cast<float*>(Vs + (size_t)G * kTcKeys * vs); // [H][16][kTcSStride]
  float* mix_s = Ss + (size_t)H * kTcRows * kTcSStride;                // [H][H]
  int* row_s = reinterpret_cast<int*>(mix_s + H * H);                  // [32]
  __shared__ int work[2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;

  // which tokens: (first token, how many)
  int t0, n_rows, seq, chunk = 0;
  if (a.split_chunk > 0) {
    seq = blockIdx.x; chunk = blockIdx.y;
    t0 = a.cu_q[seq]; n_rows = 1;
  } else {
    if (threadIdx.x == 0) {
      int left = gridDim.x - 1 - blockIdx.x, s = 0, found = -1;      // the last blocks (most keys) first
      for (; s < a.n_seqs; ++s) {
        const int len = a.cu_q[s + 1] - a.cu_q[s], nb = (len + kTcRows - 1) / kTcRows;
        if (left < nb) { found = s; break; }
        left -= nb;
      }
      work[0] = found; work[1] = left;
    }
    __syncthreads();
    seq = work[0];
    if (seq < 0) return;
    t0 = a.cu_q[seq] + work[1] * kTcRows;
    n_rows = min(kTcRows, a.cu_q[seq + 1] - t0);
  }
  const int p0 = a.positions[t0];                 // the rows' positions are p0, p0 + 1, ...
  const int p_last = p0 + n_rows - 1;
  int key_lo = (a.window > 0 && p0 + 1 > a.window) ? p0 + 1 - a.window : 0, key_hi = p_last + 1;
  if (a.split_chunk > 0) {
    key_lo = max(key_lo, chunk * a.split_chunk);
    key_hi = min(key_hi, (chunk + 1) * a.split_chunk);
    if (key_lo >= key_hi) return;
  }
  key_lo = key_lo / kTcKeys * kTcKeys;            // tiles start at multiples of 32 keys: the walk depends on positions alone
  const int* table = a.block_table + (size_t)seq * a.max_blocks;

  // queries of every head, the mixing matrix
  {
    const int chunks = d / 8;
    for (int i = threadIdx.x; i < H * kTcRows * chunks; i += kTcThreads) {
      const int c = i % chunks, r = (i / chunks) % kTcRows, h = i / (chunks * kTcRows);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < n_rows) v = *reinterpret_cast<const uint4*>(a.q + (size_t)(t0 + r) * a.q_stride + (size_t)h * d + c * 8);
      *reinterpret_cast<uint4*>(Qs + ((size_t)h * kTcRows + r) * qs + c * 8) = v;
    }
    for (int i = threadIdx.x; i < H * H; i += kTcThreads)
      mix_s[i] = a.talk != nullptr ? a.talk[i] : ((i / H == i % H) ? 1.0f : 0.0f);
  }
  const bool head_warp = warp < H;
  const int h = head_warp ? warp : 0, kvh = h / per;
  // rows gq and gq + 8 of this lane: positions, temperature
  const int pr0 = p0 + gq, pr1 = p0 + gq + 8;
  float f0 = a.scale, f1 = a.scale;
  if (a.temp_coef != 0.f) {
    f0 *= 1.0f + a.temp_coef * logf((float)((pr0 + 1) / a.temp_every) + 1.0f);
    f1 *= 1.0f + a.temp_coef * logf((float)((pr1 + 1) / a.temp_every) + 1.0f);
  }
  const float r1h = (a.r1 != nullptr && head_warp) ? a.r1[h] : 0.f, r2h = (a.r2 != nullptr && head_warp) ? a.r2[h] : 0.f;
  const float inv_cap = a.softcap > 0.f ? 1.0f / a.softcap : 0.f;
  float o[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  for (int j0 = key_lo; j0 < key_hi; j0 += kTcKeys) {
    __syncthreads();                               // the tile before is done with K, V and the scores
    if (threadIdx.x < kTcKeys) {
      const int j = j0 + threadIdx.x;
      int row = -1;
      if (j < key_hi) {
        const int page = table[j / a.page_size];
        if (page >= 0 && page < a.num_pages) row = page * a.page_size + j % a.page_size;
      }
      row_s[threadIdx.x] = row;
    }
    __syncthreads();
    {
      const int kc = d / 8, vc = dv / 8;
      for (int i = threadIdx.x; i < G * kTcKeys * (kc + vc); i += kTcThreads) {
        const int c = i % (kc + vc), jj = (i / (kc + vc)) % kTcKeys, g = i / ((kc + vc) * kTcKeys);
        const int row = row_s[jj];
        const int page = row >= 0 ? row / a.page_size : 0, place = row >= 0 ? row % a.page_size : 0;
        const size_t at = ((size_t)page * G + g) * a.page_size + place;
        if (c < kc) mix_cp_async_16(smem_u32(Ks + ((size_t)g * kTcKeys + jj) * qs + c * 8), a.k_cache + at * d + c * 8, row >= 0 ? 16 : 0);
        else mix_cp_async_16(smem_u32(Vs + ((size_t)g * kTcKeys + jj) * vs + (c - kc) * 8), a.v_cache + at * dv + (c - kc) * 8, row >= 0 ? 16 : 0);
      }
      mix_cp_async_wait_all();
    }
    __syncthreads();
    float s[4][4];
    if (head_warp) {
      // scores of head h against the 32 keys
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
      const __nv_bfloat16* qh = Qs + (size_t)h * kTcRows * qs;
      const __nv_bfloat16* kh = Ks + (size_t)kvh * kTcKeys * qs;
      for (int ks = 0; ks < d / 16; ++ks) {
        uint32_t af[4];
        ldmatrix_x4(smem_u32(qh + (size_t)(lane & 15) * qs + ks * 16 + (lane >> 4) * 8), af[0], af[1], af[2], af[3]);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(smem_u32(kh + (size_t)(np * 16 + (lane & 7) + (lane >> 4) * 8) * qs + ks * 16 + ((lane >> 3) & 1) * 8), b0, b1, b2, b3);
          mma_16816(s[2 * np], af, b0, b1);
          mma_16816(s[2 * np + 1], af, b2, b3);
        }
      }
      // shaped in 32-bit, then left for every head's mixing
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j0 + nt * 8 + 2 * tq + (e & 1);
          const int pr = (e < 2) ? pr0 : pr1;
          float v = s[nt][e] * ((e < 2) ? f0 : f1);
          if (a.softcap > 0.f) v = a.softcap * fast_tanh(v * inv_cap);
          if (a.r1 != nullptr) v -= r1h * __logf(1.0f + r2h * (float)max(pr - j, 0));
          s[nt][e] = v;
        }
      float* sh = Ss + (size_t)h * kTcRows * kTcSStride;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        *reinterpret_cast<float2*>(sh + gq * kTcSStride + nt * 8 + 2 * tq) = make_float2(s[nt][0], s[nt][1]);
        *reinterpret_cast<float2*>(sh + (gq + 8) * kTcSStride + nt * 8 + 2 * tq) = make_float2(s[nt][2], s[nt][3]);
      }
    }
    __syncthreads();
    if (head_warp) {
      // head h's mixed scores, in the layout the scores had
      const float* mh = mix_s + h * H;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
      for (int g = 0; g < H; ++g) {
        const float w = mh[g];
        const float* sg = Ss + (size_t)g * kTcRows * kTcSStride;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const float2 x0 = *reinterpret_cast<const float2*>(sg + gq * kTcSStride + nt * 8 + 2 * tq);
          const float2 x1 = *reinterpret_cast<const float2*>(sg + (gq + 8) * kTcSStride + nt * 8 + 2 * tq);
          s[nt][0] = fmaf(w, x0.x, s[nt][0]); s[nt][1] = fmaf(w, x0.y, s[nt][1]);
          s[nt][2] = fmaf(w, x1.x, s[nt][2]); s[nt][3] = fmaf(w, x1.y, s[nt][3]);
        }
      }
      // what a row may read; the running softmax
      float t0m = -INFINITY, t1m = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int c = nt * 8 + 2 * tq + (e & 1), j = j0 + c;
          const int pr = (e < 2) ? pr0 : pr1;
          const bool seen = j <= pr && j < key_hi && pr <= p_last && row_s[c] >= 0 && (a.window == 0 || j > pr - a.window) &&
                            (a.split_chunk == 0 || j >= chunk * a.split_chunk);
          if (!seen) s[nt][e] = -INFINITY;
          if (e < 2) t0m = fmaxf(t0m, s[nt][e]); else t1m = fmaxf(t1m, s[nt][e]);
        }
      t0m = fmaxf(t0m, __shfl_xor_sync(0xffffffffu, t0m, 1)); t0m = fmaxf(t0m, __shfl_xor_sync(0xffffffffu, t0m, 2));
      t1m = fmaxf(t1m, __shfl_xor_sync(0xffffffffu, t1m, 1)); t1m = fmaxf(t1m, __shfl_xor_sync(0xffffffffu, t1m, 2));
      const float n0 = fmaxf(m0, t0m), n1 = fmaxf(m1, t1m);
      const float c0 = (m0 == -INFINITY) ? 0.f : __expf(m0 - n0), c1 = (m1 == -INFINITY) ? 0.f : __expf(m1 - n1);
      m0 = n0; m1 = n1;
      l0 *= c0; l1 *= c1;
#pragma unroll
      for (int i = 0; i < DV / 8; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
      uint32_t pf[2][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const float e0 = (s[nt][0] == -INFINITY) ? 0.f : __expf(s[nt][0] - n0), e1 = (s[nt][1] == -INFINITY) ? 0.f : __expf(s[nt][1] - n0);
        const float e2 = (s[nt][2] == -INFINITY) ? 0.f : __expf(s[nt][2] - n1), e3 = (s[nt][3] == -INFINITY) ? 0.f : __expf(s[nt][3] - n1);
        l0 += e0 + e1; l1 += e2 + e3;
        pf[nt >> 1][(nt & 1) * 2] = pack_bf16(e0, e1);
        pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(e2, e3);
      }
      const __nv_bfloat16* vh = Vs + (size_t)kvh * kTcKeys * vs;
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
        for (int np = 0; np < DV / 16; ++np) {
          if (np * 16 >= dv) break;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(smem_u32(vh + (size_t)(ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * vs + np * 16 + (lane >> 4) * 8), b0, b1, b2, b3);
          mma_16816(o[2 * np], pf[ks], b0, b1);
          mma_16816(o[2 * np + 1], pf[ks], b2, b3);
        }
      }
    }
  }
  if (!head_warp) return;
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (a.split_chunk > 0) {
    // the chunk's record of the one token (row 0): max, sum, weighted values
    if (gq != 0) return;
    float* rec = a.scratch + (((size_t)seq * a.max_chunks + chunk) * H + h) * (dv + 2);
    if (tq == 0) { rec[0] = m0; rec[1] = l0; }
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) {
      if (i * 8 >= dv) break;
      rec[2 + i * 8 + 2 * tq] = o[i][0];
      rec[2 + i * 8 + 2 * tq + 1] = o[i][1];
    }
    return;
  }
  float g0 = 1.0f, g1 = 1.0f;
  if (a.sink != nullptr) {
    const float sk = a.sink[h], top0 = fmaxf(m0, sk), top1 = fmaxf(m1, sk);
    g0 = (m0 == -INFINITY) ? 0.f : __expf(m0 - top0); g1 = (m1 == -INFINITY) ? 0.f : __expf(m1 - top1);
    l0 = l0 * g0 + __expf(sk - top0); l1 = l1 * g1 + __expf(sk - top1);
  }
  g0 = l0 > 0.f ? g0 / l0 : 0.f; g1 = l1 > 0.f ? g1 / l1 : 0.f;
#pragma unroll
  for (int i = 0; i < DV / 8; ++i) {
    if (i * 8 >= dv) break;
    const int col = h * dv + i * 8 + 2 * tq;
    if (gq < n_rows) *reinterpret_cast<uint32_t*>(a.out + (size_t)(t0 + gq) * a.out_stride + col) = pack_bf16(o[i][0] * g0, o[i][1] * g0);
    if (gq + 8 < n_rows) *reinterpret_cast<uint32_t*>(a.out + (size_t)(t0 + gq + 8) * a.out_stride + col) = pack_bf16(o[i][2] * g1, o[i][3] * g1);
  }
}

// The chunks' records of a single token added in chunk order, with the sink: a block a sequence.
__global__ void __launch_bounds__(256)
attention_mix_merge_kernel(const MixTcParams a) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const int seq = blockIdx.x, H = a.nq, dv = a.dv;
  const int t = a.cu_q[seq], p = a.positions[t];
  const int lo = (a.window > 0 && p + 1 > a.window) ? p + 1 - a.window : 0;
  const int c_lo = lo / a.split_chunk, c_hi = p / a.split_chunk;
  for (int e = threadIdx.x; e < H * dv; e += blockDim.x) {
    const int h = e / dv, c = e % dv;
    float top = a.sink != nullptr ? a.sink[h] : -INFINITY;
    for (int k = c_lo; k <= c_hi; ++k)
      top = fmaxf(top, a.scratch[(((size_t)seq * a.max_chunks + k) * H + h) * (dv + 2)]);
    float l = a.sink != nullptr ? __expf(a.sink[h] - top) : 0.f, v = 0.f;
    for (int k = c_lo; k <= c_hi; ++k) {
      const float* rec = a.scratch + (((size_t)seq * a.max_chunks + k) * H + h) * (dv + 2);
      const float f = (rec[0] == -INFINITY) ? 0.f : __expf(rec[0] - top);
      l = fmaf(rec[1], f, l);
      v = fmaf(rec[2 + c], f, v);
    }
    a.out[(size_t)t * a.out_stride + e] = __float2bfloat16_rn(l > 0.f ? v / l : 0.f);
  }
}

static size_t mix_tc_smem(int nq, int nkv, int d, int dv) {
  return sizeof(__nv_bfloat16) * ((size_t)nq * kTcRows * (d + 8) + (size_t)nkv * kTcKeys * (d + 8) + (size_t)nkv * kTcKeys * (dv + 8)) +
         sizeof(float) * ((size_t)nq * kTcRows * kTcSStride + (size_t)nq * nq) + sizeof(int) * kTcKeys;
}

// Whether the tensor-core kernel takes this geometry (0 / 1).
ILB_EXPORT int ilb_attention_mix_tc_supported(int nq, int nkv, int d, int dv) {
  if (nq <= 0 || nkv <= 0 || nq % nkv || nq > kTcWarps) return 0;
  if (d <= 0 || dv <= 0 || d % 16 || dv % 16 || d > 256 || dv > 128) return 0;
  return mix_tc_smem(nq, nkv, d, dv) <= 220 * 1024 ? 1 : 0;
}

// n_blocks: the blocks of 16 tokens over all sequences (split_chunk 0), else ignored: the grid is (sequences, max_chunks).
ILB_EXPORT int ilb_attention_mix_tc(
    const void* q, void* out, const void* k_cache, const void* v_cache, const int* positions, const int* cu_q,
    const int* block_table, int max_blocks, int page_size, int num_pages, int window, float scale, int n_seqs, int n_blocks,
    int nq, int nkv, int d, int dv, int q_stride, int out_stride, const float* sink, const float* talk, const float* r1,
    const float* r2, float softcap, float temp_coef, int temp_every, int split_chunk, int max_chunks, float* scratch,
    long long scratch_floats, cudaStream_t stream) {
  ILB_REQUIRE(ilb_attention_mix_tc_supported(nq, nkv, d, dv), "attention_mix_tc: %d / %d heads of %d / %d are not served", nq, nkv, d, dv);
  ILB_REQUIRE(page_size > 0 && max_blocks > 0 && num_pages > 0 && window >= 0 && softcap >= 0.f, "attention_mix_tc: bad arguments");
  ILB_REQUIRE((r1 == nullptr) == (r2 == nullptr), "attention_mix_tc: the distance term needs both of its vectors");
  ILB_REQUIRE(temp_coef == 0.f || temp_every > 0, "attention_mix_tc: the query temperature needs a positive period");
  ILB_REQUIRE(q_stride >= nq * d && out_stride >= nq * dv && q_stride % 8 == 0 && out_stride % 2 == 0 && ((uintptr_t)q % 16 == 0) &&
              ((uintptr_t)out % 4 == 0) && ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0),
              "attention_mix_tc: rows are not aligned");
  ILB_REQUIRE(split_chunk >= 0 && (split_chunk == 0 || (split_chunk % kTcKeys == 0 && max_chunks > 0 && scratch != nullptr &&
              (long long)max_blocks * page_size <= (long long)max_chunks * split_chunk &&
              scratch_floats >= (long long)n_seqs * max_chunks * nq * (dv + 2))),
              "attention_mix_tc: the chunks do not cover the block table, or the scratch is too small");
  if (n_seqs == 0 || (split_chunk == 0 && n_blocks == 0)) return 0;
  const MixTcParams a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                      positions, cu_q, block_table, max_blocks, page_size, num_pages, window, scale, n_seqs, nq, nkv, d, dv,
                      q_stride, out_stride, sink, talk, r1, r2, softcap, temp_coef, temp_every, split_chunk, max_chunks, scratch};
  const size_t smem = mix_tc_smem(nq, nkv, d, dv);
  const dim3 grid = split_chunk > 0 ? dim3(n_seqs, max_chunks) : dim3(n_blocks);
#define ILB_TC(DV)                                                                                                        \
  do {                                                                                                                    \
    static OncePerDevice once;                                                                                            \
    if (once.first() && cudaFuncSetAttribute(attention_mix_tc_kernel<DV>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                             220 * 1024) != cudaSuccess) {                                                \
      once.forget();                                                                                                      \
      return fail("attention_mix_tc: cannot set the shared memory size: %s", cudaGetErrorString(cudaGetLastError()));     \
    }                                                                                                                     \
    ilb::launch(attention_mix_tc_kernel<DV>, grid, dim3(kTcThreads), smem, stream, a);                                    \
  } while (0)
  if (dv <= 64) ILB_TC(64); else ILB_TC(128);
#undef ILB_TC
  if (check_launch("attention_mix_tc") != 0) return -1;
  if (split_chunk > 0) {
    ilb::launch(attention_mix_merge_kernel, dim3(n_seqs), dim3(256), 0, stream, a);
    return check_launch("attention_mix_merge");
  }
  return 0;
}

ILB_DEFINE_LAST_ERROR()
