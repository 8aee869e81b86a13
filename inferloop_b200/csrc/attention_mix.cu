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
constexpr int kTcHeadScores = kTcRows * kTcKeys; // floats of a head's score tile

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
  float* scratch;                              // [n_seqs or n_tokens][max_chunks][nq][dv + 2]
  int per_token;                               // the chunks' records belong to tokens of prompt portions (else to single tokens, by sequence)
  int n_tokens;
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

__device__ __forceinline__ float mix_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float mix_lg2(float x) { float y; asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float mix_rcp(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

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
  float* Ss = reinterpret_cast<float*>(Vs + (size_t)G * kTcKeys * vs); // [H][4][32 lanes][4]: a lane's 16 scores of a head, as it holds them
  float* mix_s = Ss + (size_t)H * kTcHeadScores;                       // [H][H]
  int* row_s = reinterpret_cast<int*>(mix_s + H * H);                  // [32] row of the key in a kv head's first page place, -1: not read
  __shared__ int work[2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;

  // which tokens: (first token, how many)
  if (threadIdx.x == 0) {
    int left = gridDim.x - 1 - blockIdx.x, s = 0, found = -1;        // the last blocks (most keys) first
    for (; s < a.n_seqs; ++s) {
      const int len = a.cu_q[s + 1] - a.cu_q[s], nb = (len + kTcRows - 1) / kTcRows;
      if (left < nb) { found = s; break; }
      left -= nb;
    }
    work[0] = found; work[1] = left;
  }
  __syncthreads();
  const int seq = work[0];
  if (seq < 0) return;
  const int t0 = a.cu_q[seq] + work[1] * kTcRows;
  const int n_rows = min(kTcRows, a.cu_q[seq + 1] - t0);
  const int p0 = a.positions[t0];                 // the rows' positions are p0, p0 + 1, ...
  const int p_last = p0 + n_rows - 1;
  int key_lo = (a.window > 0 && p0 + 1 > a.window) ? p0 + 1 - a.window : 0, key_hi = p_last + 1;
  const int chunk = a.per_token ? blockIdx.y : 0;
  if (a.per_token) {                              // few blocks with many keys: block (16 tokens, chunk of keys) leaves records
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
  const bool capped = a.softcap > 0.f, shifted = a.r1 != nullptr;
  // cap tanh(s f / cap) = cap - 2 cap / (2^(s f 2 log2(e) / cap) + 1)
  if (capped) { f0 *= 2.0f * kLog2e / a.softcap; f1 *= 2.0f * kLog2e / a.softcap; }
  const float cap = a.softcap, cap2 = 2.0f * a.softcap;
  const float r1l = (shifted && head_warp) ? a.r1[h] * kLn2 : 0.f, r2h = (shifted && head_warp) ? a.r2[h] : 0.f;
  float o[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  // shared-memory addresses that no tile changes: this lane's rows of the ldmatrix loads, its scores, its copies
  const uint32_t q_addr = smem_u32(Qs + ((size_t)h * kTcRows + (lane & 15)) * qs + (lane >> 4) * 8);
  const uint32_t k_addr = smem_u32(Ks + ((size_t)kvh * kTcKeys + (lane & 7) + (lane >> 4) * 8) * qs + ((lane >> 3) & 1) * 8);
  const uint32_t k_half = 16u * qs * 2u;            // bytes from keys 0..15 to keys 16..31
  const uint32_t v_addr = smem_u32(Vs + ((size_t)kvh * kTcKeys + (lane & 7) + ((lane >> 3) & 1) * 8) * vs + (lane >> 4) * 8);
  const uint32_t v_half = 16u * vs * 2u;
  float* const s_mine = Ss + (size_t)h * kTcHeadScores + lane * 4;
  const float* const s_all = Ss + lane * 4;
  const float* const mh = mix_s + h * H;
  const int kc = d / 8, vc = dv / 8;
  const bool k_lane = lane < kc;                    // this lane copies a piece of a key row (else of a value row)
  const uint32_t copy_dst = k_lane ? smem_u32(Ks + lane * 8) : smem_u32(Vs + (lane - kc) * 8);
  const uint32_t copy_row = (k_lane ? qs : vs) * 2u;
  const __nv_bfloat16* const copy_src = k_lane ? a.k_cache + lane * 8 : a.v_cache + (lane - kc) * 8;
  const int copy_width = k_lane ? d : dv;
  const bool one_pass = kc + vc <= 32;

  for (int j0 = key_lo; j0 < key_hi; j0 += kTcKeys) {
    __syncthreads();                               // the tile before is done with K, V and the scores
    int bad = 0;
    if (threadIdx.x < kTcKeys) {
      const int j = j0 + threadIdx.x;
      int row = -1;
      if (j < key_hi) {
        const int page = table[j / a.page_size];
        if (page >= 0 && page < a.num_pages) row = page * G * a.page_size + j % a.page_size;
      }
      row_s[threadIdx.x] = row;
      bad = row < 0;
    }
    // a tile on which some (row, key) pair is not read: the diagonal's, a window's edge, a key without a page
    const bool edge = __syncthreads_or(bad) != 0 || j0 + kTcKeys - 1 > p0 || (a.window > 0 && j0 <= p_last - a.window);
    {
      for (int r = warp; r < G * kTcKeys; r += kTcWarps) {        // a warp a (kv head, key): its key row and its value row
        const int g = r / kTcKeys, jj = r % kTcKeys, row = row_s[jj];
        const size_t at = (size_t)max(row, 0) + (size_t)g * a.page_size;
        const int bytes = row >= 0 ? 16 : 0;
        if (one_pass) {                                            // a lane a piece: the row's place in shared memory is r rows down
          if (lane < kc + vc) mix_cp_async_16(copy_dst + r * copy_row, copy_src + at * copy_width, bytes);
        } else {
          for (int c = lane; c < kc + vc; c += 32) {
            if (c < kc) mix_cp_async_16(smem_u32(Ks + (size_t)r * qs + c * 8), a.k_cache + at * d + c * 8, bytes);
            else mix_cp_async_16(smem_u32(Vs + (size_t)r * vs + (c - kc) * 8), a.v_cache + at * dv + (c - kc) * 8, bytes);
          }
        }
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
#pragma unroll 2
      for (uint32_t off = 0; off < (uint32_t)d * 2u; off += 32u) {     // 16 elements of the head size a step
        uint32_t af[4], b0, b1, b2, b3;
        ldmatrix_x4(q_addr + off, af[0], af[1], af[2], af[3]);
        ldmatrix_x4(k_addr + off, b0, b1, b2, b3);
        mma_16816(s[0], af, b0, b1);
        mma_16816(s[1], af, b2, b3);
        ldmatrix_x4(k_addr + k_half + off, b0, b1, b2, b3);
        mma_16816(s[2], af, b0, b1);
        mma_16816(s[3], af, b2, b3);
      }
      // shaped in 32-bit, then left for every head's mixing
      const float d0 = (float)(pr0 - j0 - 2 * tq), d1 = d0 + 8.0f;       // distance of rows gq, gq + 8 to key j0 + 2 tq
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[nt][e] * ((e < 2) ? f0 : f1);
          if (capped) v = fmaf(-cap2, mix_rcp(mix_ex2(v) + 1.0f), cap);
          if (shifted) {
            const float dist = fmaxf(((e < 2) ? d0 : d1) - (float)(nt * 8 + (e & 1)), 0.f);
            v = fmaf(-r1l, mix_lg2(fmaf(r2h, dist, 1.0f)), v);
          }
          s[nt][e] = v;
        }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) *reinterpret_cast<float4*>(s_mine + nt * 128) = make_float4(s[nt][0], s[nt][1], s[nt][2], s[nt][3]);
    }
    __syncthreads();
    if (head_warp) {
      // head h's mixed scores, in the layout the scores had
      float2 z[4][2];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) z[nt][0] = z[nt][1] = make_float2(0.f, 0.f);
#pragma unroll 4
      for (int g = 0; g < H; ++g) {
        const float w = mh[g];
        const float2 w2 = make_float2(w, w);
        const float* sg = s_all + g * kTcHeadScores;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const float4 x = *reinterpret_cast<const float4*>(sg + nt * 128);
          z[nt][0] = __ffma2_rn(w2, make_float2(x.x, x.y), z[nt][0]);
          z[nt][1] = __ffma2_rn(w2, make_float2(x.z, x.w), z[nt][1]);
        }
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) { s[nt][0] = z[nt][0].x; s[nt][1] = z[nt][0].y; s[nt][2] = z[nt][1].x; s[nt][3] = z[nt][1].y; }
      if (edge) {
        // what a row may read
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = nt * 8 + 2 * tq + (e & 1), j = j0 + c;
            const int pr = (e < 2) ? pr0 : pr1;
            const bool seen = j <= pr && pr <= p_last && row_s[c] >= 0 && (a.window == 0 || j > pr - a.window);
            if (!seen) s[nt][e] = -INFINITY;
          }
      }
      // the running softmax, in powers of two
      float t0m = -INFINITY, t1m = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        t0m = fmaxf(t0m, fmaxf(s[nt][0], s[nt][1]));
        t1m = fmaxf(t1m, fmaxf(s[nt][2], s[nt][3]));
      }
      t0m = fmaxf(t0m, __shfl_xor_sync(0xffffffffu, t0m, 1)); t0m = fmaxf(t0m, __shfl_xor_sync(0xffffffffu, t0m, 2));
      t1m = fmaxf(t1m, __shfl_xor_sync(0xffffffffu, t1m, 1)); t1m = fmaxf(t1m, __shfl_xor_sync(0xffffffffu, t1m, 2));
      const float n0 = fmaxf(m0, t0m), n1 = fmaxf(m1, t1m);
      // a row that has seen nothing yet keeps the maximum -inf; its exponents are taken against 0 and come out 0
      const float b0 = (n0 == -INFINITY) ? 0.f : -n0 * kLog2e, b1 = (n1 == -INFINITY) ? 0.f : -n1 * kLog2e;
      const float c0 = mix_ex2(fmaf(m0, kLog2e, b0)), c1 = mix_ex2(fmaf(m1, kLog2e, b1));
      m0 = n0; m1 = n1;
      if (__any_sync(0xffffffffu, c0 != 1.0f || c1 != 1.0f)) {
        l0 *= c0; l1 *= c1;
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
      }
      uint32_t pf[2][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const float e0 = mix_ex2(fmaf(s[nt][0], kLog2e, b0)), e1 = mix_ex2(fmaf(s[nt][1], kLog2e, b0));
        const float e2 = mix_ex2(fmaf(s[nt][2], kLog2e, b1)), e3 = mix_ex2(fmaf(s[nt][3], kLog2e, b1));
        l0 += e0 + e1; l1 += e2 + e3;
        pf[nt >> 1][(nt & 1) * 2] = pack_bf16(e0, e1);
        pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(e2, e3);
      }
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
        for (int np = 0; np < DV / 16; ++np) {
          if (np * 16 >= dv) break;
          uint32_t b0v, b1v, b2v, b3v;
          ldmatrix_x4_trans(v_addr + ks * v_half + np * 32, b0v, b1v, b2v, b3v);
          mma_16816(o[2 * np], pf[ks], b0v, b1v);
          mma_16816(o[2 * np + 1], pf[ks], b2v, b3v);
        }
      }
    }
  }
  if (!head_warp) return;
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (a.per_token) {
    // the chunk's record of each of the block's tokens: max, sum, weighted values
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = gq + 8 * half;
      if (r >= n_rows) continue;
      float* rec = a.scratch + (((size_t)(t0 + r) * a.max_chunks + chunk) * H + h) * (dv + 2);
      if (tq == 0) { rec[0] = half ? m1 : m0; rec[1] = half ? l1 : l0; }
#pragma unroll
      for (int i = 0; i < DV / 8; ++i) {
        if (i * 8 >= dv) break;
        rec[2 + i * 8 + 2 * tq] = o[i][2 * half];
        rec[2 + i * 8 + 2 * tq + 1] = o[i][2 * half + 1];
      }
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

// The chunks' records of a token added in chunk order, with the sink: a thread an output element.
__global__ void __launch_bounds__(256)
attention_mix_merge_kernel(const MixTcParams a) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const int H = a.nq, dv = a.dv;
  const int t = a.per_token ? blockIdx.x : a.cu_q[blockIdx.x];       // the token, and whose records these are
  const int seq = a.per_token ? t : blockIdx.x;
  const int p = a.positions[t];
  const int lo = (a.window > 0 && p + 1 > a.window) ? p + 1 - a.window : 0;
  const int c_lo = lo / a.split_chunk, c_hi = p / a.split_chunk;
  const int e = blockIdx.y * blockDim.x + threadIdx.x;            // a thread an output element
  if (e >= H * dv) return;
  const int h = e / dv, c = e % dv;
  const float* rec = a.scratch + (((size_t)seq * a.max_chunks + c_lo) * H + h) * (dv + 2);
  const size_t step = (size_t)H * (dv + 2);
  float top = a.sink != nullptr ? a.sink[h] : -INFINITY;
#pragma unroll 4
  for (int k = c_lo; k <= c_hi; ++k) top = fmaxf(top, rec[(size_t)(k - c_lo) * step]);
  float l = a.sink != nullptr ? __expf(a.sink[h] - top) : 0.f, v = 0.f;
#pragma unroll 4
  for (int k = c_lo; k <= c_hi; ++k) {
    const float* r = rec + (size_t)(k - c_lo) * step;
    const float f = (r[0] == -INFINITY) ? 0.f : __expf(r[0] - top);
    l = fmaf(r[1], f, l);
    v = fmaf(r[2 + c], f, v);
  }
  a.out[(size_t)t * a.out_stride + e] = __float2bfloat16_rn(l > 0.f ? v / l : 0.f);
}

// ---------------------------------------------------------------------------------------------------------------
// Single tokens on the tensor cores: the HEADS are the 16 rows of the tiles, so no lane works on an empty row.
//
// Block (sequence, chunk of `split_chunk` keys) walks its keys in tiles of `key_tile` (64, 32 or 16: what fits in
// shared memory with every kv head's keys and values).  Per tile: a warp takes (kv head, 16 keys) units and forms
// all heads' scores against them (one m16n8k16 row a head), keeps the rows whose head reads that kv head, shapes
// them in 32-bit and leaves them in shared memory; then warp h mixes head h's scores out of all heads' (a lane a
// key), runs the online softmax and leaves the probabilities (bfloat16) and the factor the old sums shrink by;
// then a warp takes (kv head, 16 value columns) units, multiplies all heads' probabilities into them and keeps
// the rows of that kv head's heads.  The chunk's record (max, sum, weighted values) goes to the scratch that
// attention_mix_merge_kernel adds up, as the records of the kernel above do.
constexpr int kHdThreads = 512;
constexpr int kHdWarps = kHdThreads / 32;
constexpr int kHdRows = 16;
constexpr int kHdMaxTile = 64;
constexpr int kHdSStride = kHdMaxTile + 4;       // floats between two heads' score rows
constexpr int kHdPStride = kHdMaxTile + 8;       // bfloat16 between two heads' probability rows
constexpr int kHdUnits = 8;                      // (kv head, 16 value columns) units a warp may own: 16 * 128 / 16 / 16

template <int kt>
__global__ void __launch_bounds__(kHdThreads, 1)
attention_mix_heads_kernel(const MixTcParams a) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = a.nq, G = a.nkv, d = a.d, dv = a.dv, per = H / G;
  const int qs = d + 8, vs = dv + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);       // [16][qs], rows from H on are zero
  __nv_bfloat16* Ks = Qs + (size_t)kHdRows * qs;                        // [G][kt][qs]
  __nv_bfloat16* Vs = Ks + (size_t)G * kt * qs;                         // [G][kt][vs]
  __nv_bfloat16* Ps = Vs + (size_t)G * kt * vs;                         // [16][kHdPStride]
  float* Ss = reinterpret_cast<float*>(Ps + kHdRows * kHdPStride);      // [16][kHdSStride]
  float* mix_s = Ss + kHdRows * kHdSStride;                             // [H][H]
  float* corr_s = mix_s + H * H;                                        // [16]
  int* row_s = reinterpret_cast<int*>(corr_s + kHdRows);                // [kHdMaxTile]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  const int seq = blockIdx.x, chunk = blockIdx.y;
  const int t = a.cu_q[seq], p = a.positions[t];
  int key_lo = (a.window > 0 && p + 1 > a.window) ? p + 1 - a.window : 0;
  key_lo = max(key_lo, chunk * a.split_chunk);
  const int key_hi = min(p + 1, (chunk + 1) * a.split_chunk);
  if (key_lo >= key_hi) return;
  const int* table = a.block_table + (size_t)seq * a.max_blocks;

  {
    const int chunks = d / 8;
    for (int i = threadIdx.x; i < kHdRows * chunks; i += kHdThreads) {
      const int c = i % chunks, h = i / chunks;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (h < H) v = *reinterpret_cast<const uint4*>(a.q + (size_t)t * a.q_stride + (size_t)h * d + c * 8);
      *reinterpret_cast<uint4*>(Qs + (size_t)h * qs + c * 8) = v;
    }
    for (int i = threadIdx.x; i < H * H; i += kHdThreads)
      mix_s[i] = a.talk != nullptr ? a.talk[i] : ((i / H == i % H) ? 1.0f : 0.0f);
    for (int i = threadIdx.x; i < kHdRows * kHdPStride; i += kHdThreads) Ps[i] = __float2bfloat16_rn(0.f);
  }
  float f = a.scale;
  if (a.temp_coef != 0.f) f *= 1.0f + a.temp_coef * logf((float)((p + 1) / a.temp_every) + 1.0f);
  const float inv_cap = a.softcap > 0.f ? 1.0f / a.softcap : 0.f;
  // the two heads whose rows this lane holds in an accumulator
  const int ha = gq, hb = gq + 8;
  const int ga = ha < H ? ha / per : -1, gb = hb < H ? hb / per : -1;
  const float r1a = (a.r1 != nullptr && ha < H) ? a.r1[ha] : 0.f, r2a = (a.r1 != nullptr && ha < H) ? a.r2[ha] : 0.f;
  const float r1b = (a.r1 != nullptr && hb < H) ? a.r1[hb] : 0.f, r2b = (a.r1 != nullptr && hb < H) ? a.r2[hb] : 0.f;
  const int v_units = G * (dv / 16);
  float acc[kHdUnits][2][4];
#pragma unroll
  for (int i = 0; i < kHdUnits; ++i)
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][n][e] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;          // of head `warp`, the same in every lane
  // addresses that no tile changes: this lane's piece of a copied row, its rows of the ldmatrix loads
  const int kc = d / 8, vc = dv / 8;
  const bool k_lane = lane < kc, one_pass = kc + vc <= 32;
  const uint32_t copy_dst = k_lane ? smem_u32(Ks + lane * 8) : smem_u32(Vs + (lane - kc) * 8);
  const uint32_t copy_row = (k_lane ? qs : vs) * 2u;
  const __nv_bfloat16* const copy_src = k_lane ? a.k_cache + lane * 8 : a.v_cache + (lane - kc) * 8;
  const int copy_width = k_lane ? d : dv;
  const uint32_t q_addr = smem_u32(Qs + (size_t)(lane & 15) * qs + (lane >> 4) * 8);
  const uint32_t k_lane_addr = smem_u32(Ks + (size_t)((lane & 7) + (lane >> 4) * 8) * qs + ((lane >> 3) & 1) * 8);
  const uint32_t p_addr = smem_u32(Ps + (size_t)(lane & 15) * kHdPStride + (lane >> 4) * 8);
  uint32_t v_unit[kHdUnits];                     // where unit i's value columns start, for this lane
#pragma unroll
  for (int i = 0; i < kHdUnits; ++i) {
    const int u = warp + i * kHdWarps, g = u / (dv / 16), np = u % (dv / 16);
    v_unit[i] = smem_u32(Vs + ((size_t)g * kt + (lane & 7) + ((lane >> 3) & 1) * 8) * vs + np * 16 + (lane >> 4) * 8);
  }

  for (int j0 = key_lo / kt * kt; j0 < key_hi; j0 += kt) {
    __syncthreads();                              // the tile before is done with everything in shared memory
    if (threadIdx.x < kt) {
      const int j = j0 + threadIdx.x;
      int row = -1;
      if (j >= key_lo && j < key_hi) {
        const int page = table[j / a.page_size];
        if (page >= 0 && page < a.num_pages) row = page * G * a.page_size + j % a.page_size;     // of kv head 0
      }
      row_s[threadIdx.x] = row;
    }
    __syncthreads();
    for (int r = warp; r < G * kt; r += kHdWarps) {          // a warp a (kv head, key): its key row and its value row
      const int g = r / kt, jj = r % kt, row = row_s[jj];
      const size_t at = (size_t)max(row, 0) + (size_t)g * a.page_size;
      const int bytes = row >= 0 ? 16 : 0;
      if (one_pass) {                                          // a lane a piece: the row's place in shared memory is r rows down
        if (lane < kc + vc) mix_cp_async_16(copy_dst + r * copy_row, copy_src + at * copy_width, bytes);
      } else {
        for (int c = lane; c < kc + vc; c += 32) {
          if (c < kc) mix_cp_async_16(smem_u32(Ks + (size_t)r * qs + c * 8), a.k_cache + at * d + c * 8, bytes);
          else mix_cp_async_16(smem_u32(Vs + (size_t)r * vs + (c - kc) * 8), a.v_cache + at * dv + (c - kc) * 8, bytes);
        }
      }
    }
    mix_cp_async_wait_all();
    __syncthreads();
    // all heads' scores against (kv head, 16 keys); the rows of that kv head's heads are kept and shaped
    for (int u = warp; u < G * (kt / 16); u += kHdWarps) {
      const int g = u / (kt / 16), np = u % (kt / 16);
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t k_addr = k_lane_addr + (uint32_t)(g * kt + np * 16) * qs * 2u;
#pragma unroll 2
      for (uint32_t off = 0; off < (uint32_t)d * 2u; off += 32u) {
        uint32_t af[4], b0, b1, b2, b3;
        ldmatrix_x4(q_addr + off, af[0], af[1], af[2], af[3]);
        ldmatrix_x4(k_addr + off, b0, b1, b2, b3);
        mma_16816(s0, af, b0, b1);
        mma_16816(s1, af, b2, b3);
      }
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const bool first = e < 2;
          if ((first ? ga : gb) != g) continue;
          const int jj = np * 16 + n * 8 + 2 * tq + (e & 1);
          float v = (n == 0 ? s0[e] : s1[e]) * f;
          if (a.softcap > 0.f) v = a.softcap * fast_tanh(v * inv_cap);
          if (a.r1 != nullptr) v -= (first ? r1a : r1b) * __logf(1.0f + (first ? r2a : r2b) * (float)max(p - (j0 + jj), 0));
          Ss[(first ? ha : hb) * kHdSStride + jj] = v;
        }
    }
    __syncthreads();
    if (warp < H) {
      const float* mh = mix_s + warp * H;
      float z[2], e[2];
      float top = -INFINITY;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int jj = lane + 32 * i;
        z[i] = -INFINITY;
        if (jj < kt && row_s[jj] >= 0) {
          float x = 0.f;
          for (int g = 0; g < H; ++g) x = fmaf(mh[g], Ss[g * kHdSStride + jj], x);
          z[i] = x;
        }
        top = fmaxf(top, z[i]);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
      const float m_new = fmaxf(m_run, top);
      const float c = (m_run == -INFINITY) ? 0.f : __expf(m_run - m_new);
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        e[i] = (z[i] == -INFINITY) ? 0.f : __expf(z[i] - m_new);
        sum += e[i];
        const int jj = lane + 32 * i;
        if (jj < kt) Ps[warp * kHdPStride + jj] = __float2bfloat16_rn(e[i]);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      l_run = l_run * c + sum;
      m_run = m_new;
      if (lane == 0) corr_s[warp] = c;
    } else if (lane == 0) {
      corr_s[warp] = 0.f;
    }
    __syncthreads();
    // all heads' probabilities into (kv head, 16 value columns)
    {
      const float ca = corr_s[ha], cb = corr_s[hb];
#pragma unroll
      for (int i = 0; i < kHdUnits; ++i) {
        const int u = warp + i * kHdWarps;
        if (u >= v_units) break;
#pragma unroll
        for (int n = 0; n < 2; ++n) { acc[i][n][0] *= ca; acc[i][n][1] *= ca; acc[i][n][2] *= cb; acc[i][n][3] *= cb; }
#pragma unroll
        for (int ks = 0; ks < kt / 16; ++ks) {
          uint32_t pf[4], b0, b1, b2, b3;
          ldmatrix_x4(p_addr + ks * 32, pf[0], pf[1], pf[2], pf[3]);
          ldmatrix_x4_trans(v_unit[i] + ks * 16 * vs * 2, b0, b1, b2, b3);
          mma_16816(acc[i][0], pf, b0, b1);
          mma_16816(acc[i][1], pf, b2, b3);
        }
      }
    }
  }
  // the chunk's record of every head
  if (warp < H && lane == 0) {
    float* rec = a.scratch + (((size_t)seq * a.max_chunks + chunk) * H + warp) * (dv + 2);
    rec[0] = m_run; rec[1] = l_run;
  }
#pragma unroll
  for (int i = 0; i < kHdUnits; ++i) {
    const int u = warp + i * kHdWarps;
    if (u >= v_units) break;
    const int g = u / (dv / 16), np = u % (dv / 16);
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const int col = 2 + np * 16 + n * 8 + 2 * tq;
      if (ga == g) {
        float* rec = a.scratch + (((size_t)seq * a.max_chunks + chunk) * H + ha) * (dv + 2);
        rec[col] = acc[i][n][0]; rec[col + 1] = acc[i][n][1];
      }
      if (gb == g) {
        float* rec = a.scratch + (((size_t)seq * a.max_chunks + chunk) * H + hb) * (dv + 2);
        rec[col] = acc[i][n][2]; rec[col + 1] = acc[i][n][3];
      }
    }
  }
}

static size_t mix_heads_smem(int nq, int nkv, int d, int dv, int kt) {
  return sizeof(__nv_bfloat16) * ((size_t)kHdRows * (d + 8) + (size_t)nkv * kt * (d + 8) + (size_t)nkv * kt * (dv + 8) +
                                  (size_t)kHdRows * kHdPStride) +
         sizeof(float) * ((size_t)kHdRows * kHdSStride + (size_t)nq * nq + kHdRows) + sizeof(int) * kHdMaxTile;
}

// The key tile of the kernel for single tokens: the largest of 64, 32, 16 that fits and divides the chunk.
static int mix_heads_tile(int nq, int nkv, int d, int dv, int split_chunk) {
  for (int kt = kHdMaxTile; kt >= 16; kt /= 2)
    if (split_chunk % kt == 0 && mix_heads_smem(nq, nkv, d, dv, kt) <= 200 * 1024) return kt;
  return 0;
}

static size_t mix_tc_smem(int nq, int nkv, int d, int dv) {
  return sizeof(__nv_bfloat16) * ((size_t)nq * kTcRows * (d + 8) + (size_t)nkv * kTcKeys * (d + 8) + (size_t)nkv * kTcKeys * (dv + 8)) +
         sizeof(float) * ((size_t)nq * kTcHeadScores + (size_t)nq * nq) + sizeof(int) * kTcKeys;
}

// Whether the tensor-core kernel takes this geometry (0 / 1).
ILB_EXPORT int ilb_attention_mix_tc_supported(int nq, int nkv, int d, int dv) {
  if (nq <= 0 || nkv <= 0 || nq % nkv || nq > kTcWarps) return 0;
  if (d <= 0 || dv <= 0 || d % 16 || dv % 16 || d > 256 || dv > 128) return 0;
  if (mix_heads_smem(nq, nkv, d, dv, 16) > 200 * 1024) return 0;
  return mix_tc_smem(nq, nkv, d, dv) <= 220 * 1024 ? 1 : 0;
}

// n_blocks: the blocks of 16 tokens over all sequences.  split_chunk > 0 without per_token: single tokens, the grid is
// (sequences, max_chunks).  With per_token: prompt portions whose blocks are few and whose keys are many; the grid is
// (n_blocks, max_chunks) and a second launch adds every token's records.
ILB_EXPORT int ilb_attention_mix_tc(
    const void* q, void* out, const void* k_cache, const void* v_cache, const int* positions, const int* cu_q,
    const int* block_table, int max_blocks, int page_size, int num_pages, int window, float scale, int n_seqs, int n_blocks,
    int nq, int nkv, int d, int dv, int q_stride, int out_stride, const float* sink, const float* talk, const float* r1,
    const float* r2, float softcap, float temp_coef, int temp_every, int split_chunk, int max_chunks, float* scratch,
    long long scratch_floats, int per_token, int n_tokens, cudaStream_t stream) {
  ILB_REQUIRE(ilb_attention_mix_tc_supported(nq, nkv, d, dv), "attention_mix_tc: %d / %d heads of %d / %d are not served", nq, nkv, d, dv);
  ILB_REQUIRE(page_size > 0 && max_blocks > 0 && num_pages > 0 && window >= 0 && softcap >= 0.f, "attention_mix_tc: bad arguments");
  ILB_REQUIRE((r1 == nullptr) == (r2 == nullptr), "attention_mix_tc: the distance term needs both of its vectors");
  ILB_REQUIRE(temp_coef == 0.f || temp_every > 0, "attention_mix_tc: the query temperature needs a positive period");
  ILB_REQUIRE(q_stride >= nq * d && out_stride >= nq * dv && q_stride % 8 == 0 && out_stride % 2 == 0 && ((uintptr_t)q % 16 == 0) &&
              ((uintptr_t)out % 4 == 0) && ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0),
              "attention_mix_tc: rows are not aligned");
  ILB_REQUIRE(split_chunk >= 0 && (split_chunk == 0 || (split_chunk % kTcKeys == 0 && max_chunks > 0 && scratch != nullptr)),
              "attention_mix_tc: chunks are multiples of %d keys and need a scratch", kTcKeys);
  ILB_REQUIRE(split_chunk == 0 || per_token != 0 || ((long long)max_blocks * page_size <= (long long)max_chunks * split_chunk &&
              scratch_floats >= (long long)n_seqs * max_chunks * nq * (dv + 2)),
              "attention_mix_tc: the chunks do not cover the block table, or the scratch is too small");
  ILB_REQUIRE(per_token == 0 || (split_chunk > 0 && n_tokens > 0 && n_blocks > 0 &&
              scratch_floats >= (long long)n_tokens * max_chunks * nq * (dv + 2)),
              "attention_mix_tc: records by token need chunks, the blocks and a scratch for every token");
  if (n_seqs == 0 || (split_chunk == 0 && n_blocks == 0)) return 0;
  const MixTcParams a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                      positions, cu_q, block_table, max_blocks, page_size, num_pages, window, scale, n_seqs, nq, nkv, d, dv,
                      q_stride, out_stride, sink, talk, r1, r2, softcap, temp_coef, temp_every, split_chunk, max_chunks, scratch,
                      per_token, n_tokens};
  if (split_chunk > 0 && !per_token) {
    // single tokens: the heads are the rows of the tiles; the chunks' records are added by a second launch
    const int kt = mix_heads_tile(nq, nkv, d, dv, split_chunk);
    ILB_REQUIRE(kt > 0, "attention_mix_tc: no key tile fits chunks of %d keys", split_chunk);
#define ILB_HD(KT)                                                                                                        \
  do {                                                                                                                    \
    static OncePerDevice once;                                                                                            \
    if (once.first() && cudaFuncSetAttribute(attention_mix_heads_kernel<KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                             200 * 1024) != cudaSuccess) {                                                \
      once.forget();                                                                                                      \
      return fail("attention_mix_tc: cannot set the shared memory size: %s", cudaGetErrorString(cudaGetLastError()));     \
    }                                                                                                                     \
    ilb::launch(attention_mix_heads_kernel<KT>, dim3(n_seqs, max_chunks), dim3(kHdThreads),                               \
                mix_heads_smem(nq, nkv, d, dv, KT), stream, a);                                                           \
  } while (0)
    if (kt == 64) ILB_HD(64); else if (kt == 32) ILB_HD(32); else ILB_HD(16);
#undef ILB_HD
    if (check_launch("attention_mix_heads") != 0) return -1;
    ilb::launch(attention_mix_merge_kernel, dim3(n_seqs, (nq * dv + 255) / 256), dim3(256), 0, stream, a);
    return check_launch("attention_mix_merge");
  }
  const size_t smem = mix_tc_smem(nq, nkv, d, dv);
  const dim3 grid = per_token ? dim3(n_blocks, max_chunks) : dim3(n_blocks);
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
  if (per_token) {
    ilb::launch(attention_mix_merge_kernel, dim3(n_tokens, (nq * dv + 255) / 256), dim3(256), 0, stream, a);
    return check_launch("attention_mix_merge");
  }
  return 0;
}

ILB_DEFINE_LAST_ERROR()
