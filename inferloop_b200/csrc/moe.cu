// Routed feed-forward ("mixture of experts"): what lies around the experts' matrix products.
//
//   logits   z[T, E (+ 1)] = x W_router^T in 32-bit (a skinny product: a warp per token)
//   route    router logits z[T, E] (32-bit) -> scores (sigmoid of each logit, or softmax over the
//            experts), the `top` best experts of every token (ties to the lower index) and their
//            weights (the chosen scores, optionally divided by their sum)
//   plan     the (token, choice) pairs sorted by expert: every expert's rows start at a multiple
//            of `block_rows`, so that a block of rows belongs to one expert; pos[pair] = row,
//            block_expert[block] = expert or -1
//   gather   a[pos[pair], :] = x[token of the pair, :] (times the pair's weight, when the weight
//            multiplies the expert's input); rows that hold no pair are left as they are: a row
//            of a product depends on no other row, and nobody reads theirs
//   combine  y[t, :] += sum over the token's choices, in choice order, of (weight *) out[pos, :]
//            (+ gate[t] * shared[t, :], gate = sigmoid of a logit, for an expert every token uses)
//
// Scores, weights and the sums are 32-bit.  Nothing here depends on the host knowing how many
// tokens an expert got: every size is the worst case, and blocks without an expert are skipped,
// so a recorded launch sequence can be replayed for another batch.
#include <math.h>
#include "common.cuh"

using namespace ilb;

constexpr int kMaxExpertsPerLane = 16;      // experts <= 32 * this
constexpr int kMaxTop = 32;

__device__ __forceinline__ float sigmoid_stable(float x) {
  if (x >= 0.f) return 1.0f / (1.0f + expf(-x));
  const float e = expf(x);
  return e / (1.0f + e);
}

// Router logits: out[t, e] = x[t, :] . w[e, :] in 32-bit for a few rows of w (the experts, and a
// gate's row riding along).  A block of four warps owns one token and kLogitRows rows of w:
// threads take consecutive pieces of eight features; a piece is one chain of fused multiply-adds
// from zero, the pieces of a thread are added with the rounding error of every addition carried
// along in a second word (two-sum), the lanes meet in a butterfly sum and the warps in a fixed order.  The order of a logit's sum
// depends on the width alone, and its error stays near that of eight terms, not of the width.
constexpr int kLogitRows = 4;

template <typename T> struct Piece8;
template <> struct Piece8<float> {
  __device__ static __forceinline__ void load(const float* p, float (&f)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
};
template <> struct Piece8<__nv_bfloat16> {
  __device__ static __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
  }
};

template <typename T>
__global__ void __launch_bounds__(128)
moe_logits_kernel(const T* __restrict__ x, const T* __restrict__ w, float* __restrict__ out, int n_tokens, int rows, int width,
                  int vec) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  __shared__ float part_sum[4][kLogitRows];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const T* xr = x + (size_t)t * width;
  const int e0 = blockIdx.y * kLogitRows;
  float acc[kLogitRows], lost[kLogitRows];
#pragma unroll
  for (int r = 0; r < kLogitRows; ++r) { acc[r] = 0.f; lost[r] = 0.f; }
  auto add = [&](int r, float part) {
    const float sum = __fadd_rn(acc[r], part);
    const float bp = __fsub_rn(sum, acc[r]);
    lost[r] = __fadd_rn(lost[r], __fadd_rn(__fsub_rn(acc[r], __fsub_rn(sum, bp)), __fsub_rn(part, bp)));
    acc[r] = sum;
  };
  if (vec) {
    for (int i = threadIdx.x * 8; i < width; i += 1024) {
      float xv[8];
      Piece8<T>::load(xr + i, xv);
#pragma unroll
      for (int r = 0; r < kLogitRows; ++r) {
        if (e0 + r >= rows) break;
        float wv[8];
        Piece8<T>::load(w + (size_t)(e0 + r) * width + i, wv);
        float part = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) part = fmaf(xv[k], wv[k], part);
        add(r, part);
      }
    }
  } else {
    for (int i = threadIdx.x; i < width; i += 128) {
      const float xv = to_float(xr[i]);
#pragma unroll
      for (int r = 0; r < kLogitRows; ++r)
        if (e0 + r < rows) add(r, __fmul_rn(xv, to_float(w[(size_t)(e0 + r) * width + i])));
    }
  }
#pragma unroll
  for (int r = 0; r < kLogitRows; ++r) {
    const float v = warp_sum(__fadd_rn(acc[r], lost[r]));
    if (lane == 0) part_sum[warp][r] = v;
  }
  __syncthreads();
  if (threadIdx.x < kLogitRows && e0 + threadIdx.x < rows) {
    const int r = threadIdx.x;
    out[(size_t)t * rows + e0 + r] = (part_sum[0][r] + part_sum[1][r]) + (part_sum[2][r] + part_sum[3][r]);
  }
}

// x: [T, width], w: [rows, width], both of `dtype`; out: [T, rows] 32-bit.
ILB_EXPORT int ilb_moe_logits(const void* x, const void* w, int dtype, float* out, int n_tokens, int rows, int width,
                              cudaStream_t stream) {
  ILB_REQUIRE(n_tokens >= 0 && rows > 0 && width > 0, "moe_logits: bad sizes");
  ILB_REQUIRE((rows + kLogitRows - 1) / kLogitRows <= 65535, "moe_logits: too many rows");
  if (n_tokens == 0) return 0;
  const dim3 grid(n_tokens, (rows + kLogitRows - 1) / kLogitRows);
  const int vec = (width % 8 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0)) ? 1 : 0;
  if (dtype == kF32)
    ilb::launch(moe_logits_kernel<float>, grid, dim3(128), 0, stream, (const float*)x, (const float*)w, out, n_tokens, rows, width, vec);
  else if (dtype == kBF16)
    ilb::launch(moe_logits_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, out,
                n_tokens, rows, width, vec);
  else
    return fail("moe_logits: unknown dtype %d", dtype);
  return check_launch("moe_logits");
}

// One warp per token.
__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int ld, int n_tokens, int experts, int top,
                 int softmax, int renormalize, int* __restrict__ choice, float* __restrict__ weight,
                 const float* __restrict__ correction, int groups, int keep, float out_scale, float renorm_eps) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= n_tokens) return;
  const float* z = logits + (size_t)t * ld;
  float s[kMaxExpertsPerLane];
  float zmax = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxExpertsPerLane; ++i) {
    const int e = lane + 32 * i;
    s[i] = e < experts ? (bias != nullptr ? z[e] + bias[e] : z[e]) : -INFINITY;
    zmax = fmaxf(zmax, s[i]);
  }
  if (softmax) {
    zmax = warp_max(zmax);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      s[i] = e < experts ? expf(s[i] - zmax) : -INFINITY;
      if (e < experts) sum += s[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i)
      if (lane + 32 * i < experts) s[i] = s[i] / sum;
  } else {
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i)
      if (lane + 32 * i < experts) s[i] = sigmoid_stable(s[i]);
  }
  // What the experts are ranked by: the scores, or the scores plus a stored correction (the weights below are the
  // scores themselves either way).  With groups, only experts of the `keep` groups of neighbours whose best ranked
  // member is largest can be chosen (ties to the lower group).
  float c[kMaxExpertsPerLane];
#pragma unroll
  for (int i = 0; i < kMaxExpertsPerLane; ++i) {
    const int e = lane + 32 * i;
    c[i] = (e < experts && correction != nullptr) ? s[i] + correction[e] : s[i];
  }
  if (groups > 1 && keep < groups) {
    const int per = experts / groups;
    float mine = -INFINITY;                // lane g: group g's best member
    for (int g = 0; g < groups; ++g) {
      float m = -INFINITY;
#pragma unroll
      for (int i = 0; i < kMaxExpertsPerLane; ++i) {
        const int e = lane + 32 * i;
        if (e < experts && e / per == g) m = fmaxf(m, c[i]);
      }
      m = warp_max(m);
      if (lane == g) mine = m;
    }
    unsigned allowed = 0u;
    for (int j = 0; j < keep; ++j) {
      float best = mine;
      int best_g = (lane < groups && mine != -INFINITY) ? lane : 0x7fffffff;
      if (best_g == 0x7fffffff) best = -INFINITY;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
        if (ob > best || (ob == best && og < best_g)) { best = ob; best_g = og; }
      }
      if (best_g == 0x7fffffff) break;
      allowed |= 1u << best_g;
      if (lane == best_g) mine = -INFINITY;
    }
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      if (e < experts && !((allowed >> (e / per)) & 1u)) c[i] = -INFINITY;
    }
  }
  float chosen_w = 0.f, total = 0.f;     // lane j keeps the j-th choice
  int chosen_e = 0;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      if (e < experts && (c[i] > best || (c[i] == best && e < best_e)) && c[i] != -INFINITY) { best = c[i]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if (best_e == 0x7fffffff) { best_e = 0; best = 0.f; }      // (non-finite logits: keep the indices in range)
    float score = 0.f;                                          // the winner's score, from the lane that holds it
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i)
      if (lane + 32 * i == best_e) { score = s[i]; c[i] = -INFINITY; }      // taken
    score = __shfl_sync(0xffffffffu, score, best_e & 31);
    if (score == -INFINITY) score = 0.f;
    if (lane == j) { chosen_w = score; chosen_e = best_e; }
    total += score;
  }
  if (lane < top) {
    choice[(size_t)t * top + lane] = chosen_e;
    weight[(size_t)t * top + lane] = (renormalize ? chosen_w / (total + renorm_eps) : chosen_w) * out_scale;
  }
}

ILB_EXPORT int ilb_moe_max_experts() { return 32 * kMaxExpertsPerLane; }
ILB_EXPORT int ilb_moe_max_top() { return kMaxTop; }

// logits: [T, ld] 32-bit, the first `experts` columns are the router's.  choice / weight: [T, top].
// bias: [experts] added to the logits first, or null.  correction: [experts] added to the scores for the ranking
// alone, or null.  groups > 1 with keep < groups: only the best `keep` of `groups` equal groups of neighbouring
// experts can be chosen.  Weights: the chosen scores (divided by their sum + renorm_eps when renormalize) * out_scale.
ILB_EXPORT int ilb_moe_route(const float* logits, const float* bias, int ld, int n_tokens, int experts, int top, int softmax,
                             int renormalize, int* choice, float* weight, const float* correction, int groups, int keep,
                             float out_scale, float renorm_eps, cudaStream_t stream) {
  ILB_REQUIRE(groups >= 1 && groups <= 32 && experts % groups == 0 && keep >= 1 && keep <= groups,
              "moe_route: %d groups (at most 32, dividing %d experts), %d kept", groups, experts, keep);
  ILB_REQUIRE(top <= (experts / groups) * keep, "moe_route: top %d exceeds the %d experts of the kept groups", top, (experts / groups) * keep);
  ILB_REQUIRE(n_tokens >= 0 && experts > 0 && experts <= 32 * kMaxExpertsPerLane, "moe_route: %d experts (at most %d)", experts,
              32 * kMaxExpertsPerLane);
  ILB_REQUIRE(top > 0 && top <= experts && top <= kMaxTop, "moe_route: top %d of %d experts (at most %d)", top, experts, kMaxTop);
  ILB_REQUIRE(ld >= experts, "moe_route: row stride too small");
  if (n_tokens == 0) return 0;
  ilb::launch(moe_route_kernel, dim3((n_tokens + 3) / 4), dim3(128), 0, stream, logits, bias, ld, n_tokens, experts, top, softmax,
              renormalize, choice, weight, correction, groups, keep, out_scale, renorm_eps);
  return check_launch("moe_route");
}

// One CTA.  counts and offsets of the experts live in shared memory.
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ choice, int n_pairs, int experts, int block_rows, int max_rows,
                int* __restrict__ pos, int* __restrict__ block_expert) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  extern __shared__ int sh[];
  int* count = sh;                 // [experts]
  int* start = sh + experts;       // [experts + 1], in rows
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  for (int b = threadIdx.x; b < max_rows / block_rows; b += blockDim.x) block_expert[b] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = choice[p];
    pos[p] = (e >= 0 && e < experts) ? atomicAdd(&count[e], 1) : -1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < experts; ++e) {
      start[e] = at;
      at += (count[e] + block_rows - 1) / block_rows * block_rows;
    }
    start[experts] = at;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x)
    for (int b = start[e] / block_rows; b < start[e + 1] / block_rows; ++b) block_expert[b] = e;
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = choice[p];
    if (pos[p] < 0) continue;
    pos[p] = start[e] + pos[p];
  }
}

// Rows that n_pairs pairs over `experts` experts can need when every expert's rows are padded to
// a multiple of block_rows.
static inline long long plan_rows(long long n_pairs, int experts, int block_rows) {
  const long long most_experts = n_pairs < experts ? n_pairs : experts;
  const long long rows = n_pairs + most_experts * (block_rows - 1);
  return (rows + block_rows - 1) / block_rows * block_rows;
}
ILB_EXPORT long long ilb_moe_plan_rows(long long n_pairs, int experts, int block_rows) { return plan_rows(n_pairs, experts, block_rows); }

// choice: [n_pairs]; pos: [n_pairs]; block_expert: [max_rows / block_rows];
// max_rows >= ilb_moe_plan_rows(n_pairs, experts, block_rows), a multiple of block_rows.
ILB_EXPORT int ilb_moe_plan(const int* choice, int n_pairs, int experts, int block_rows, int max_rows, int* pos,
                            int* block_expert, cudaStream_t stream) {
  ILB_REQUIRE(n_pairs >= 0 && experts > 0 && block_rows > 0, "moe_plan: bad sizes");
  ILB_REQUIRE(max_rows % block_rows == 0 && max_rows >= plan_rows(n_pairs, experts, block_rows), "moe_plan: %d rows are too few",
              max_rows);
  ILB_REQUIRE((size_t)(2 * experts + 1) * sizeof(int) <= 48 * 1024, "moe_plan: too many experts");
  if (n_pairs == 0) return 0;
  ilb::launch(moe_plan_kernel, dim3(1), dim3(1024), (size_t)(2 * experts + 1) * sizeof(int), stream, choice, n_pairs, experts,
              block_rows, max_rows, pos, block_expert);
  return check_launch("moe_plan");
}

template <typename T>
__global__ void __launch_bounds__(128)
moe_gather_kernel(const T* __restrict__ x, const float* __restrict__ weight, const int* __restrict__ pos, int top, int width,
                  T* __restrict__ out) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const int p = blockIdx.x;
  const int row = pos[p];
  if (row < 0) return;
  T* o = out + (size_t)row * width;
  const T* src = x + (size_t)(p / top) * width;
  const int step = blockDim.x * gridDim.y, first = blockIdx.y * blockDim.x + threadIdx.x;    // the row is dealt over gridDim.y blocks
  if (weight == nullptr) {
    for (int i = first; i < width; i += step) o[i] = src[i];
  } else {
    const float w = weight[p];
    for (int i = first; i < width; i += step) o[i] = from_float<T>(w * to_float(src[i]));
  }
}

// x: [T, width]; pos: [n_pairs] (pair t * top + j belongs to token t); out: [rows, width];
// weight (may be null): [n_pairs].
ILB_EXPORT int ilb_moe_gather(const void* x, int dtype, const float* weight, const int* pos, int n_pairs, int top, int width,
                              void* out, cudaStream_t stream) {
  ILB_REQUIRE(n_pairs >= 0 && top > 0 && width > 0, "moe_gather: bad sizes");
  if (n_pairs == 0) return 0;
  const int ny = n_pairs >= 512 ? 1 : (width + 511) / 512 < 16 ? (width + 511) / 512 : 16;     // few pairs: more blocks per row
  if (dtype == kF32)
    ilb::launch(moe_gather_kernel<float>, dim3(n_pairs, ny), dim3(128), 0, stream, (const float*)x, weight, pos, top, width, (float*)out);
  else if (dtype == kBF16)
    ilb::launch(moe_gather_kernel<__nv_bfloat16>, dim3(n_pairs, ny), dim3(128), 0, stream, (const __nv_bfloat16*)x, weight, pos, top,
                width, (__nv_bfloat16*)out);
  else
    return fail("moe_gather: unknown dtype %d", dtype);
  return check_launch("moe_gather");
}

__global__ void __launch_bounds__(128)
moe_combine_kernel(const float* __restrict__ routed, const int* __restrict__ pos, const float* __restrict__ weight, int top,
                   const float* __restrict__ shared, const float* __restrict__ gate_logit, int gate_ld, int width,
                   float* __restrict__ y) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const int t = blockIdx.x;
  __shared__ int rows[kMaxTop];
  __shared__ float ws[kMaxTop];
  if (threadIdx.x < top) {
    rows[threadIdx.x] = pos[(size_t)t * top + threadIdx.x];
    ws[threadIdx.x] = weight != nullptr ? weight[(size_t)t * top + threadIdx.x] : 1.0f;
  }
  __syncthreads();
  float gate = 1.0f;
  if (shared != nullptr && gate_logit != nullptr) gate = sigmoid_stable(gate_logit[(size_t)t * gate_ld]);
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < width; i += blockDim.x * gridDim.y) {
    float v = 0.f;
    for (int j = 0; j < top; ++j)
      if (rows[j] >= 0) v = fmaf(ws[j], routed[(size_t)rows[j] * width + i], v);
    if (shared != nullptr) v = fmaf(gate, shared[(size_t)t * width + i], v);
    y[(size_t)t * width + i] += v;
  }
}

// routed: [rows, width] 32-bit, the experts' outputs; pos: [T, top]; weight: [T, top] or null
// (the weight was applied to the input); shared: [T, width] 32-bit or null; gate_logit: a column
// of a 32-bit matrix with row stride gate_ld, or null (no gate); y: [T, width] 32-bit, added to.
ILB_EXPORT int ilb_moe_combine(const float* routed, const int* pos, const float* weight, int top, const float* shared,
                               const float* gate_logit, int gate_ld, int n_tokens, int width, float* y, cudaStream_t stream) {
  ILB_REQUIRE(n_tokens >= 0 && top > 0 && top <= kMaxTop && width > 0, "moe_combine: bad sizes");
  if (n_tokens == 0) return 0;
  const int ny = n_tokens >= 512 ? 1 : (width + 255) / 256 < 32 ? (width + 255) / 256 : 32;    // few tokens: more blocks per row
  ilb::launch(moe_combine_kernel, dim3(n_tokens, ny), dim3(128), 0, stream, routed, pos, weight, top, shared, gate_logit, gate_ld, width, y);
  return check_launch("moe_combine");
}

ILB_DEFINE_LAST_ERROR()
